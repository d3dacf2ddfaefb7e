#!/usr/bin/env python
"""Benchmark of the dense-contraction inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C1..C5]

Workload (default): configuration C2 of BASELINE.json, the fp32 CNN on [256,3,32,32] -- the largest
fp32 configuration the reference's own generated CPU code runs. One step = one Session::infer over
one batch of seeded synthetic input. Multi-GPU: one process per GPU (torchrun), each rank runs the
same per-GPU batch (weak scaling, the batch dimension is sharded, weights replicated, no
collective on the data path); `value` is the whole-job samples/s, timed on the device, max over
ranks.

`--impl reference` times the reference's own emitted CPU code (oracle/_ref, built from the
unmodified reference generator; OpenBLAS with all host threads) on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD_DESC = {
    "C1": "fp32 MLP 64-128-128-10, batch 1024",
    "C2": "fp32 CNN [256,3,32,32]: 3x(Conv3x3+Relu), 2xMaxPool, Gemm 4096-10",
    "C3": "int8 MLP 512-1024-1024-256, batch 8192",
    "C4": "FP8 E4M3 Gemm chain 4x(K=N=4096), M=65536",
    "C5": "int8 calorimeter CNN [16384,1,64,64]",
}
DTYPE = {"C1": "f32", "C2": "f32", "C3": "u8", "C4": "e4m3", "C5": "u8"}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


def tensor_peak_tflops(workload, pk):
    """Dense tensor-core peak of the workload's arithmetic, derived from the measured bf16 number:
    FP8 and INT8 = 2 x bf16, TF32 = bf16 / 2, fp32 through 3 TF32 products = TF32 / 3."""
    bf16 = pk["bf16_tflops"]
    return {"C1": bf16 / 6, "C2": bf16 / 6, "C3": bf16 * 2, "C4": bf16 * 2, "C5": bf16 * 2}[workload]


class ClockSampler:
    """SM clock and throttle reasons of this rank's GPU, read through NVML every 5 ms by a thread for the
    whole run (reading only; nothing is set). stop() keeps the samples that fall inside the timed windows
    (device-timed steps and end-to-end steps). A timed region shorter than a few samples is followed by
    `load()` -- the same step replayed for a fraction of a second, outside any timing -- so that the
    clock under this load is still on record."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        import threading
        self.windows, self.rows, self.err = [], [], None
        self._stop = threading.Event()
        self.handle = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            self.nv = pynvml
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception as e:  # no NVML: the line says so instead of inventing a clock
            self.err = f"NVML unavailable: {type(e).__name__}"

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                clk = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.rows.append((time.time(), clk, mask))
            except Exception as e:
                self.err = f"NVML read failed: {type(e).__name__}"
                return
            time.sleep(0.005)

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def samples_in_windows(self):
        return [r for r in self.rows if any(t0 <= r[0] <= t1 for t0, t1 in self.windows)]

    def load(self, step_fn, seconds=0.4):
        """Replays the step for `seconds` (untimed) when the timed windows hold fewer than 3 samples."""
        if self.handle is None or len(self.samples_in_windows()) >= 3:
            return False
        import torch
        t0 = time.time()
        while time.time() - t0 < seconds:
            for _ in range(50):
                step_fn()
            torch.cuda.synchronize()
        self.windows = [(t0, time.time())]
        return True

    def stop(self, scope="timed windows"):
        if self.handle is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[self.err or "NVML unavailable"], samples=0, scope=scope)
        self._stop.set()
        self.thread.join(timeout=1.0)
        inside = self.samples_in_windows()
        reasons = sorted({name for r in inside for name, bit in self.REASONS if r[2] & bit})
        return dict(sm_mhz=float(np.median([r[1] for r in inside])) if inside else None, sm_max_mhz=self.sm_max,
                    reasons=reasons, samples=len(inside), scope=scope)


# DRAM traffic per launch of the dominant kernels, from ncu captures (profiles/): bytes read + written.
NCU_TRAFFIC = {
    # profiles/umma_conv3x3_f32_C2.md: conv2 of C2 at the full batch of 256: 16.84 MB read, 0 written
    # (the pooled output stays in L2)
    ("C2", "conv:p1"): 16.84e6,
}


def build_workload(workload, batch=None):
    """The configuration at its full size, or (profiling aid, --batch) at a reduced batch / row count."""
    from sofie_b200 import configs
    if workload == "C4":
        return configs.gemm_chain_fp8(rows=batch) if batch else configs.gemm_chain_fp8()
    return configs.BUILDERS[workload](batch=batch) if batch else configs.BUILDERS[workload]()


# ------------------------------------------------------------------------------------ reference arm
def reference_arm(args, rank, world):
    if rank != 0:
        return 0
    from oracle import build_ref, ref_runner, run_model
    from sofie_b200 import configs
    case = {"C1": "ref_c1", "C2": "ref_c2"}.get(args.workload)
    m, x = build_workload(args.workload)
    cores = os.cpu_count() or 1
    if case and ref_runner.available():
        kind = "reference"
        ref_runner.set_threads(cores)
        n_out = int(np.prod([m.batch()] + [10]))

        def step():
            return ref_runner.infer(case, x, n_out)
        sample = f"full {args.workload} batch of {m.batch()} per step, reference-emitted C++ at -O3 + OpenBLAS ({ref_runner.blas_config()})"
        samples_per_step = m.batch()
    else:
        # int8 / FP8 configurations do not exist in the reference: the oracle port is timed on a bounded sample
        kind = "port"
        nb = {"C3": 1024, "C4": 64, "C5": 32}.get(args.workload, m.batch())
        m2, x2 = (configs.BUILDERS[args.workload](batch=nb) if args.workload != "C4"
                  else configs.gemm_chain_fp8(rows=nb))
        scales = run_model.calibrate_fp8_scales(m2, x2) if args.workload == "C4" else None

        def step():
            return run_model.run(m2, x2, fp8_scales=scales)
        sample = f"{nb} of {m.batch()} samples per step, plain-C oracle port, pthreads"
        samples_per_step = nb
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = samples_per_step * args.steps / dt
    line = dict(metric="samples/s", value=value, unit="samples/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1e3 * dt / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype=DTYPE[args.workload], data="synthetic", impl="reference",
                config=dict(workload=f"{args.workload}: {WORKLOAD_DESC[args.workload]}", batch_per_step=samples_per_step),
                cpu_baseline=dict(value=value, unit="samples/s", cores=cores, kind=kind, sample=sample),
                e2e=dict(value=value, unit="samples/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))
    return 0


def cpu_baseline(workload, budget_s=12.0):
    """Reference CPU code (or the oracle port) on the host cores, bounded sample; rank 0, N=1 only."""
    from oracle import ref_runner, run_model
    from sofie_b200 import configs
    case = {"C1": "ref_c1", "C2": "ref_c2"}.get(workload)
    cores = os.cpu_count() or 1
    if case and ref_runner.available():
        m, x = build_workload(workload)
        ref_runner.set_threads(cores)
        n_out = m.batch() * 10
        fn, nb, kind = (lambda: ref_runner.infer(case, x, n_out)), m.batch(), "reference"
        what = f"reference-emitted C++ -O3 + OpenBLAS, {cores} threads, full batch {nb}"
    else:
        nb = {"C1": 1024, "C2": 64, "C3": 1024, "C4": 64, "C5": 32}[workload]
        m, x = (configs.BUILDERS[workload](batch=nb) if workload != "C4" else configs.gemm_chain_fp8(rows=nb))
        scales = run_model.calibrate_fp8_scales(m, x) if workload == "C4" else None
        fn, kind = (lambda: run_model.run(m, x, fp8_scales=scales)), "port"
        what = f"plain-C oracle port, {cores} pthreads, {nb} samples per call"
    fn()
    fn()
    t0 = time.perf_counter()
    calls = 0
    while calls < 3 or (time.perf_counter() - t0 < budget_s and calls < 200):
        fn()
        calls += 1
    dt = time.perf_counter() - t0
    return dict(value=nb * calls / dt, unit="samples/s", cores=cores, kind=kind, sample=f"{calls} calls in {dt:.1f} s; {what}")


# ------------------------------------------------------------------------------------ our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOAD_DESC))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layer-times", action="store_true", help="also time every step of the plan alone (adds layer_ms to the line)")
    ap.add_argument("--batch", type=int, default=None, help="reduced batch / rows for ncu captures (not a benchmark configuration)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, rank, world)

    import torch
    import torch.distributed as dist

    from sofie_b200 import configs, runner

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libSOFIE_cuda has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    os.environ["SOFIE_CUDA_DEVICE"] = str(local_rank)  # the emitted Session reads its device from here
    clocks = ClockSampler(local_rank)
    m, x = build_workload(args.workload, args.batch)
    scales = None
    if args.workload == "C4":
        # static FP8 activation scales from an fp32 run of the chain on a 512-row slice (setup)
        scales = configs.calibrate_fp8_scales(m, x[:512])
    sess = runner.Session(m, device=local_rank, fp8_scales=scales, use_graph=True)
    x_pinned = torch.from_numpy(x).pin_memory()
    x_dev = x_pinned.cuda(non_blocking=True)
    torch.cuda.synchronize()
    sess.capture(x_dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    # ---- device-timed steps, inputs resident in HBM, L2 flushed between steps ----
    for _ in range(args.warmup):
        sess.replay()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    w0 = time.time()
    for i in range(args.steps):
        flush.zero_()
        starts[i].record()
        sess.replay()
        ends[i].record()
    barrier()
    clocks.window(w0, time.time())
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    # ---- end to end through the emitted C++ Session (ONNX -> Parse -> Generate -> g++ -> Session::infer):
    #      pinned host input -> device, captured graph, device -> host output, every step.
    y_host = torch.empty(tuple(sess.static_out.shape), dtype=sess.static_out.dtype).pin_memory()
    e2e_path = "emitted C++ Session::infer"
    from sofie_b200 import generated
    # C4's weights (4 x 16.8 MB of E4M3) go through the binary side file; the text form is kept for the rest
    gen = generated.session_from_model(m, f"bench_{args.workload.lower()}_{m.batch()}", binary=(args.workload == "C4"),
                                       fp8_scales=scales)

    def e2e_step():
        gen.infer_ptr(x_pinned.data_ptr(), y_host.data_ptr())
    for _ in range(args.warmup):
        e2e_step()
    barrier()
    w0 = time.time()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    clocks.window(w0, time.time())
    barrier()
    if args.workload in ("C1", "C2"):
        # the two paths must agree (same kernels, same weights)
        ref = sess.static_out.float().cpu().numpy().ravel()
        got = y_host.float().numpy().ravel()
        assert np.abs(ref - got).max() <= 1e-5 * max(np.abs(ref).max(), 1e-30), "emitted Session and Python mirror disagree"

    # ---- dominant kernel, timed alone with events on the launching stream ----
    # The event pair sits INSIDE a captured graph (flush, record, kernel, record), so the interval is
    # the kernel's time on the device and holds none of the host's launch latency.
    dom = max((s for s in sess.steps if s.flops), key=lambda s: s.flops)
    t = sess._run_steps(x_dev)  # materialise the inputs of every step

    def device_time_ms(fn, reps):
        for _ in range(3):
            fn(t)
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True, external=True)
        b = torch.cuda.Event(enable_timing=True, external=True)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            flush.zero_()
            a.record()
            fn(t)
            b.record()
        tot = 0.0
        for _ in range(reps):
            g.replay()
            torch.cuda.synchronize()
            tot += a.elapsed_time(b)
        return tot / reps

    k_ms = device_time_ms(dom.fn, max(10, min(args.steps, 50)))
    layer_ms = None
    if args.layer_times:
        # every step of the plan timed alone (cold L2), to see where a step's time goes
        layer_ms = {st.name: round(device_time_ms(st.fn, 5), 5) for st in sess.steps}
    extended = clocks.load(sess.replay)
    clk = clocks.stop("timed windows" if not extended else
                      "0.4 s of replays of the same step right after the timed region (it was shorter than three samples)")

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    batch = m.batch()
    pk = peaks()
    kflops = dom.flops * batch
    tpeak = tensor_peak_tflops(args.workload, pk)
    achieved = kflops / (k_ms * 1e-3) / 1e12
    line = dict(
        metric="samples/s", value=world * batch * args.steps / (dev_ms * 1e-3), unit="samples/s", n_gpus=world,
        steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype=DTYPE[args.workload], data="synthetic",
        config=dict(workload=f"{args.workload}: {WORKLOAD_DESC[args.workload]}" + (f" [reduced to batch {args.batch}]" if args.batch else ""),
                    batch_per_gpu=batch,
                    parallelism=f"batch-sharded x{world}, weights replicated, no collective",
                    l2="flushed between timed steps (256 MiB memset outside the event pairs)",
                    launch="CUDA graph replay of the infer() kernel sequence", e2e_path=e2e_path),
        tflops=m.flops_per_sample * batch * world * args.steps / (dev_ms * 1e-3) / 1e12,
        e2e=dict(value=world * batch * args.steps / (e2e_ms * 1e-3), unit="samples/s",
                 h2d_bytes_per_step=int(x_pinned.numel() * x_pinned.element_size()),
                 d2h_bytes_per_step=int(y_host.numel() * y_host.element_size())),
        gpu_launches=sess.kernel_launches() * args.steps,
        roofline=dict(bound="tensor", kernel=dom.name, achieved=achieved, peak=tpeak, unit="TFLOP/s", frac=achieved / tpeak,
                      traffic=NCU_TRAFFIC.get((args.workload, dom.name)), kernel_ms=k_ms, flops_per_launch=kflops,
                      peak_basis=f"{pk['source']} bf16 {pk['bf16_tflops']} TFLOP/s scaled to the dtype"),
        clocks=clk,
    )
    if layer_ms is not None:
        line["layer_ms"] = layer_ms
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
