#!/usr/bin/env python
"""Benchmark of the dense-contraction inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C1..C5] [--batch B]

Headline workload (default): configuration C5 of the benchmark definition, the int8 calorimeter CNN on
[16384,1,64,64] -- the configuration that is sharded across 1/2/4/8 GPUs. One step = one
Session::infer over the whole batch. Everything timed runs through the C++ Session the generator emits
(ONNX bytes -> RModelParser_ONNX::Parse -> RModel::Generate -> g++ -> Session): `value` replays the Session's own
captured CUDA graph with the input resident on the device (Session::RunResident, device-timed with CUDA events
on the Session's stream, L2 flushed between steps); `e2e` calls Session::infer(float*) with a pinned host buffer,
so every step holds the host->device copy of the input and the read-back of the result. A large input is uploaded
in parts with the model's leading operators launched per part (what infer() does by itself); `value` then uses the
Session of the same model emitted with Options::kSingleUpload, whose graph runs every operator once over the batch.

Multi-GPU (torchrun, one process per GPU): the batch of 16384 images is split into contiguous shards, one per
rank; every rank builds its own Session for its shard (weights replicated), there is no collective on the data
path, and the job's throughput is the whole batch over the slowest rank's time: strong scaling.

With one GPU the line also carries `per_config` (C1..C5 at the sizes of the benchmark definition) and `large_batch` (C1 and C3 at 2^18
rows, C2 at 8192 images), each with value, e2e from pinned and from pageable memory, the dominant contraction's
roofline fraction and -- where the CPU baseline leg ran -- the comparison of the GPU result with the CPU result
on the baseline's sample, and `hbm_ops`: the memory-bound operators of the path (Relu, Softmax, MaxPool, (de)quantise,
layout change ...) called alone on tensors larger than L2, in GB/s against the measured copy bandwidth.

`--impl reference` times the CPU side on the same workload: the reference's own emitted C++ (oracle/_ref,
-O3 + OpenBLAS, all host threads) for the fp32 configurations C1/C2; for the quantised configurations, which
the reference does not have, the plain-C oracle port on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import time
import traceback
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD_DESC = {
    "C1": "fp32 MLP 64-128-128-10, batch 1024",
    "C2": "fp32 CNN [256,3,32,32]: 3x(Conv3x3+Relu), 2xMaxPool, Gemm 4096-10",
    "C3": "int8 MLP 512-1024-1024-256, batch 8192",
    "C4": "FP8 E4M3 Gemm chain 4x(K=N=4096), M=65536",
    "C5": "int8 calorimeter CNN [16384,1,64,64]: 4x(QLinearConv3x3+Relu+MaxPool), QLinearMatMul 2048-256-2",
}
DTYPE = {"C1": "f32", "C2": "f32", "C3": "u8", "C4": "e4m3", "C5": "u8"}
OUT_PER_SAMPLE = {"C1": 10, "C2": 10, "C3": 256, "C4": 4096, "C5": 2}
# samples per call of the CPU side where the whole batch would take minutes
CPU_SAMPLE = {"C1": 1024, "C2": 256, "C3": 1024, "C4": 64, "C5": 32}


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


def dram_traffic_table():
    """profiles/dram_traffic.md: DRAM bytes per launch of the dominant kernels from ncu captures, one table row per
    kernel: | workload | operator | batch | bytes | scales | source |."""
    rows = []
    p = ROOT / "profiles" / "dram_traffic.md"
    if not p.exists():
        return rows
    for ln in p.read_text().splitlines():
        cells = [c.strip() for c in ln.strip().strip("|").split("|")]
        if len(cells) == 6 and cells[0] in WORKLOAD_DESC:
            try:
                rows.append(dict(workload=cells[0], op=cells[1], batch=int(cells[2]), bytes=float(cells[3]),
                                 scales=cells[4].lower().startswith("y"), source=cells[5]))
            except ValueError:
                pass
    return rows


def dram_traffic(workload, title, batch):
    for r in dram_traffic_table():
        if r["workload"] == workload and r["op"] in title:
            if r["batch"] == batch:
                return r["bytes"], f"{r['source']} (ncu capture at this batch)"
            if r["scales"]:
                return r["bytes"] * batch / r["batch"], f"{r['source']} (ncu capture at batch {r['batch']}, scaled by the batch: every byte is read once per image)"
    return None, None


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
            for _ in range(20):
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


def pin_to_gpu_numa_node(local_rank):
    """Restricts this rank to the host cores of its GPU's NUMA node (the copy of the input starts in host memory
    this process touches; a remote node halves its rate). Reads sysfs only; returns what was done for the record."""
    try:
        import torch
        p = torch.cuda.get_device_properties(local_rank)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        base = Path("/sys/bus/pci/devices") / bus
        node = int((base / "numa_node").read_text())
        cpus = set()
        for part in (base / "local_cpulist").read_text().strip().split(","):
            if part:
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if not use or use == allowed:
            return dict(numa_node=node, pinned=False, cores=len(allowed))
        os.sched_setaffinity(0, use)
        return dict(numa_node=node, pinned=True, cores=len(use))
    except Exception as e:
        return dict(numa_node=None, pinned=False, why=f"{type(e).__name__}")


def place_host_memory_near_gpu(local_rank, record):
    """Where sysfs names no NUMA node for the GPU (a container), asks NVML which host cores and which memory node are
    nearest to it and (a) restricts this process to those of them it is allowed to run on, (b) makes that node the preferred
    one for this process's page allocations (set_mempolicy, MPOL_PREFERRED: a hint, allocation elsewhere still succeeds), so
    that the pinned input buffer allocated next lies on the GPU's side of the host. Process-local; nothing outlasts the process.
    Adds what it did to `record`."""
    try:
        import ctypes
        import platform
        import pynvml
        import torch
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        allowed = os.sched_getaffinity(0)
        try:
            words = (max(allowed) // 64) + 1
            mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
            cpus = {64 * w + b for w in range(words) for b in range(64) if (int(mask[w]) >> b) & 1}
            use = cpus & allowed
            record["nvml_cpus"] = len(cpus)
            if use and use != allowed:
                os.sched_setaffinity(0, use)
                record.update(pinned=True, cores=len(use))
        except Exception as e:
            record["nvml_cpu_affinity"] = type(e).__name__
        try:
            nodes = pynvml.nvmlDeviceGetMemoryAffinity(h, 1, pynvml.NVML_AFFINITY_SCOPE_NODE)
            node_mask = int(nodes[0])
            record["nvml_mem_nodes"] = node_mask
            if node_mask and platform.machine() == "x86_64":
                libc = ctypes.CDLL(None, use_errno=True)
                m = ctypes.c_ulong(node_mask)
                rc = libc.syscall(238, 1, ctypes.byref(m), 65)   # set_mempolicy(MPOL_PREFERRED, &mask, maxnode)
                record["mempolicy"] = "preferred" if rc == 0 else f"errno {ctypes.get_errno()}"
        except Exception as e:
            record["nvml_mem_affinity"] = type(e).__name__
    except Exception as e:
        record["nvml"] = type(e).__name__
    return record


# ------------------------------------------------------------------------------------ workloads
def build_workload(workload, batch=None, with_input=True):
    """The configuration at its full size, or at another batch / row count (large-batch entries, shards, captures)."""
    from sofie_b200 import configs
    if workload == "C4":
        return configs.gemm_chain_fp8(rows=batch, with_input=with_input) if batch else configs.gemm_chain_fp8(with_input=with_input)
    return configs.BUILDERS[workload](batch=batch, with_input=with_input) if batch else configs.BUILDERS[workload](with_input=with_input)


def shard_workload(workload, batch, rank, world):
    """This rank's share of the seeded workload: the model sized for its contiguous shard of the batch (the weights
    are drawn before the input, so they do not depend on the batch) and the shard's rows of the full input."""
    from sofie_b200 import configs, sharding
    m_full, x_full = build_workload(workload, batch)
    scales = configs.calibrate_fp8_scales(m_full, x_full[:512]) if workload == "C4" else None
    if world == 1:
        return m_full, x_full, scales, m_full.batch()
    b, e = sharding.shard_bounds(m_full.batch(), world, rank)
    m, _ = build_workload(workload, e - b, with_input=False)
    return m, np.ascontiguousarray(x_full[b:e]), scales, m_full.batch()


# ------------------------------------------------------------------------------------ CPU side
def cpu_runner(workload, x_full, fp8_scales=None):
    """(callable, samples per call, kind, description, rows it computes) of the CPU implementation: the reference's
    own emitted code on the full batch where it exists (C1, C2), the oracle port on the first rows otherwise."""
    from oracle import ref_runner, run_model
    case = {"C1": "ref_c1", "C2": "ref_c2"}.get(workload)
    cores = os.cpu_count() or 1
    full_batch = {"C1": 1024, "C2": 256}.get(workload)
    if case and ref_runner.available() and x_full.shape[0] == full_batch:
        ref_runner.set_threads(cores)
        n_out = x_full.shape[0] * OUT_PER_SAMPLE[workload]
        return (lambda: ref_runner.infer(case, x_full, n_out)), x_full.shape[0], "reference", \
            f"reference-emitted C++ -O3 + OpenBLAS ({ref_runner.blas_config()}), {cores} threads, full batch {x_full.shape[0]}", cores
    nb = min(CPU_SAMPLE[workload], x_full.shape[0])
    m, _ = build_workload(workload, nb, with_input=False)
    xs = np.ascontiguousarray(x_full[:nb])
    return (lambda: run_model.run(m, xs, fp8_scales=fp8_scales)), nb, "port", \
        f"plain-C oracle port, {cores} pthreads, first {nb} samples of the batch per call", cores


def cpu_baseline(workload, x_full, gpu_out, fp8_scales=None, budget_s=10.0):
    """Times the CPU side on a bounded sample and, as the checker, compares its result with the GPU result for the
    same rows (gpu_out: the emitted Session's output for the whole batch)."""
    fn, nb, kind, what, cores = cpu_runner(workload, x_full, fp8_scales)
    ref = np.asarray(fn(), np.float32).ravel()
    fn()
    t0 = time.perf_counter()
    calls = 0
    while calls < 2 or (time.perf_counter() - t0 < budget_s and calls < 100):
        fn()
        calls += 1
    dt = time.perf_counter() - t0
    got = np.asarray(gpu_out, np.float32).ravel()[: ref.size]
    if workload in ("C3", "C5"):
        parity = dict(rows=nb, rule="bit-exact", ok=bool(np.array_equal(got.view(np.uint32), ref.view(np.uint32))))
    else:
        err = float(np.abs(got - ref).max() / max(float(np.abs(ref).max()), 1e-30))
        tol = 2e-2 if workload == "C4" else 1e-5
        parity = dict(rows=nb, rule=f"max|d|/max|ref| <= {tol}", err=err, ok=bool(err <= tol))
    return dict(value=nb * calls / dt, unit="samples/s", cores=cores, kind=kind, sample=f"{calls} calls in {dt:.1f} s; {what}"), parity


def reference_arm(args, rank, world):
    if rank != 0:
        return 0
    from sofie_b200 import configs
    m, x = build_workload(args.workload, args.batch)
    scales = configs.calibrate_fp8_scales(m, x[:512]) if args.workload == "C4" else None
    fn, nb, kind, what, cores = cpu_runner(args.workload, x, scales)
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    value = nb * args.steps / dt
    line = dict(metric="samples/s", value=value, unit="samples/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1e3 * dt / args.steps, higher_is_better=True, scaling="strong", vs_baseline=None,
                dtype=DTYPE[args.workload], data="synthetic", impl="reference",
                config=dict(workload=f"{args.workload}: {WORKLOAD_DESC[args.workload]}", samples_per_step=nb),
                cpu_baseline=dict(value=value, unit="samples/s", cores=cores, kind=kind, sample=f"{args.steps} steps of {nb} samples; {what}"),
                e2e=dict(value=value, unit="samples/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------ GPU side
class Measured:
    """One workload on this rank's GPU through the emitted C++ Session."""

    def __init__(self, workload, batch, rank, world, local_rank, tag=""):
        import torch
        from sofie_b200 import capi, generated
        self.torch, self.capi = torch, capi
        self.workload, self.world = workload, world
        self.model, self.x, self.scales, self.total_batch = shard_workload(workload, batch, rank, world)
        self.shard = self.model.batch()
        name = f"bench_{workload.lower()}_{self.shard}{tag}"
        binary = workload == "C4"   # 4 x 16.8 MB of E4M3 weights: the raw side file, not 800 MB of text
        self.gen = generated.session_from_model(self.model, name, binary=binary, fp8_scales=self.scales)
        self.pipelined = "void LaunchHead(int part)" in self.gen.hxx.read_text()
        # A large input is uploaded in parts and the model's leading operators run per part (infer(), `e2e`). With the input
        # already on the device there is nothing to overlap: `value` replays the graph of the same model emitted with
        # Options::kSingleUpload, every operator once over the whole batch.
        self.resident = self.gen
        if self.pipelined:
            self.resident = generated.session_from_model(self.model, name + "_single", binary=binary, fp8_scales=self.scales, pipelined=False)
        self.plan = generated.launch_plan(self.resident.hxx)
        self.x_pinned = torch.from_numpy(self.x).pin_memory()
        self.y_host = torch.empty(self.gen.out_elems, dtype=torch.float32).pin_memory()
        stream = C.c_void_p()
        capi.call("sofie_cuda_ctx_stream", self.resident.ctx, C.byref(stream))
        self.stream = torch.cuda.ExternalStream(stream.value, device=torch.device("cuda", local_rank))
        self.local_rank = local_rank
        # the first call runs the launch sequence eagerly and captures it, the second replays the graph
        for sess in {id(self.gen): self.gen, id(self.resident): self.resident}.values():
            sess.infer_ptr(self.x_pinned.data_ptr(), self.y_host.data_ptr())
            sess.infer_ptr(self.x_pinned.data_ptr(), self.y_host.data_ptr())

    def infer(self):
        self.gen.infer_ptr(self.x_pinned.data_ptr(), self.y_host.data_ptr())

    def kernel_launches(self):
        """Kernels of this library launched per device-timed step: one per libSOFIE_cuda call of the emitted Launch()
        (the skinny split-K GEMM launches two)."""
        return sum(len(p["calls"]) for p in self.plan)

    def device_timed(self, steps, warmup, flush, barrier, clocks=None):
        torch = self.torch
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                self.resident.run_resident()
            barrier()
            w0 = time.time()
            for i in range(steps):
                flush.zero_()
                starts[i].record()
                self.resident.run_resident()
                ends[i].record()
            barrier()
        if clocks:
            clocks.window(w0, time.time())
        self.capi.call("sofie_cuda_ctx_check", self.resident.ctx)
        return sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    def end_to_end(self, steps, warmup, barrier, clocks=None, pageable=False):
        if pageable:
            x_plain = np.array(self.x, copy=True)   # ordinary (pageable) host memory, as a SOFIE user's buffer is
            y_plain = np.empty(self.gen.out_elems, np.float32)
            xp, yp = x_plain.ctypes.data, y_plain.ctypes.data
        else:
            xp, yp = self.x_pinned.data_ptr(), self.y_host.data_ptr()
        for _ in range(warmup):
            self.gen.infer_ptr(xp, yp)
        barrier()
        w0 = time.time()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.gen.infer_ptr(xp, yp)
        dt = time.perf_counter() - t0
        if clocks:
            clocks.window(w0, time.time())
        barrier()
        return dt * 1e3

    def h2d_ms(self, reps=5):
        """The input copy alone (pinned host -> device), device-timed: what end-to-end cannot go below."""
        torch = self.torch
        dst = torch.empty_like(self.x_pinned, device=torch.device("cuda", self.local_rank))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = 1e30
        for _ in range(reps):
            a.record()
            dst.copy_(self.x_pinned, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            best = min(best, a.elapsed_time(b))
        return best

    def operator_times(self, flush, reps):
        """Milliseconds per operator of Launch(), from the library's device timers: a second Session of the same model
        (uploaded in one piece, so that every operator is part of Launch()) with the timers on, run `reps` times
        after an L2 flush; the operators follow each other as in a real step (an operator finds its input where
        the previous one left it)."""
        from sofie_b200 import generated
        torch, capi = self.torch, self.capi
        os.environ["SOFIE_CUDA_TIMERS"] = "1"
        try:
            name = f"bench_{self.workload.lower()}_{self.shard}_single"
            timed = generated.session_from_model(self.model, name, binary=self.workload == "C4", fp8_scales=self.scales,
                                                 pipelined=False if self.pipelined else None)
        finally:
            del os.environ["SOFIE_CUDA_TIMERS"]
        plan = generated.launch_plan(timed.hxx)
        timed.infer_ptr(self.x_pinned.data_ptr(), self.y_host.data_ptr())
        timed.infer_ptr(self.x_pinned.data_ptr(), self.y_host.data_ptr())
        stream = C.c_void_p()
        capi.call("sofie_cuda_ctx_stream", timed.ctx, C.byref(stream))
        ext = torch.cuda.ExternalStream(stream.value, device=torch.device("cuda", self.local_rank))
        n = len(plan)
        acc = np.zeros(n)
        buf = (C.c_float * n)()
        count = C.c_int()
        for _ in range(reps):
            with torch.cuda.stream(ext):
                flush.zero_()
            timed.run_resident()
            capi.call("sofie_cuda_ctx_timers_read", timed.ctx, buf, n, C.byref(count))
            if count.value != n:
                raise RuntimeError(f"{count.value} timer intervals for {n} operators")
            acc += np.frombuffer(buf, np.float32, n)
        timed.close()
        return [dict(p, ms=float(t / reps)) for p, t in zip(plan, acc)]

    def output(self):
        return self.y_host.numpy()

    def close(self):
        self.gen.close()
        if self.resident is not self.gen:
            self.resident.close()


NOMINAL_BF16_TFLOPS = 2250.0  # B200 dense bf16, datasheet; the other dtypes scale from it as they do from the measured number


def roofline_of(workload, ops, shard_batch, pk):
    dom = max(ops, key=lambda o: o["flops"])
    tpeak = tensor_peak_tflops(workload, pk)
    achieved = dom["flops"] / (dom["ms"] * 1e-3) / 1e12
    traffic, source = dram_traffic(workload, dom["title"], shard_batch)
    nominal = tpeak / pk["bf16_tflops"] * NOMINAL_BF16_TFLOPS
    return dict(bound="tensor", kernel=dom["title"], achieved=achieved, peak=tpeak, unit="TFLOP/s", frac=achieved / tpeak,
                peak_nominal=nominal, frac_nominal=achieved / nominal,
                traffic=traffic, traffic_source=source, kernel_ms=dom["ms"], flops_per_launch=dom["flops"],
                peak_basis=f"{pk['source']} bf16 {pk['bf16_tflops']} TFLOP/s (burst) scaled to the dtype: fp32 as 3xTF32 = bf16/6, int8 and FP8 = 2 x bf16",
                timing="the library's device timers (CUDA events around every operator of the emitted Launch(), in a captured graph), mean of the repetitions, each after an L2 flush")


def memory_bound_ops(ops, model, pk):
    """Achieved GB/s of the non-contraction kernels that stand alone in the plan (quantise, pool, softmax ...)."""
    out = []
    x_elems = int(np.prod(model.input_shape))
    for o in ops:
        if o["flops"] == 0 and o["ms"] > 0 and o["calls"] and o["calls"][0] in ("sofie_cuda_quantize_u8", "sofie_cuda_quantize_e4m3_f32"):
            nbytes = x_elems * 5  # float in, one byte out
            out.append(dict(kernel=o["title"], bytes=nbytes, ms=o["ms"], gbs=nbytes / (o["ms"] * 1e-3) / 1e9,
                            frac=nbytes / (o["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]))
    return out


def standalone_hbm_ops(torch, pk, reps=5):
    """Achieved GB/s of the memory-bound operators of the path, each called alone through the C ABI on tensors larger than
    L2 (256-512 MB of traffic per call), CUDA events on the launching stream, median of `reps` after one warm-up call.
    bytes = what the operator has to read plus what it has to write."""
    from sofie_b200 import ops
    dev = "cuda"
    n = 1 << 26                                                   # 64 Mi elements: 256 MB of floats
    x = torch.randn(n, device=dev)
    y = torch.randn(n, device=dev)
    img = x.view(1024, 16, 64, 64)
    q = ops.quantize_u8(x, 0.02, 128)
    cases = [
        ("Relu (sofie_cuda_relu_f32)", lambda: ops.relu_f32(x), 8 * n),
        ("Sigmoid (sofie_cuda_unary_f32)", lambda: ops.unary_f32(x, "Sigmoid"), 8 * n),
        ("Add (sofie_cuda_binary_f32)", lambda: ops.binary_f32(x, y, "Add"), 12 * n),
        ("Softmax over 1000 classes (sofie_cuda_softmax_f32)", lambda: ops.softmax_f32(x[: 65536 * 1000].view(65536, 1000)), 8 * 65536 * 1000),
        ("Softmax over 10 classes (sofie_cuda_softmax_f32)", lambda: ops.softmax_f32(x[: (1 << 22) * 10].view(1 << 22, 10)), 8 * (1 << 22) * 10),
        ("MaxPool 2x2 fp32 NCHW (sofie_cuda_pool2d_f32)", lambda: ops.pool2d_f32(img), 5 * n),
        ("QuantizeLinear to uint8 (sofie_cuda_quantize_u8)", lambda: ops.quantize_u8(x, 0.02, 128), 5 * n),
        ("DequantizeLinear from uint8 (sofie_cuda_dequantize_u8)", lambda: ops.dequantize_u8(q, 0.02, 128), 5 * n),
        ("Quantize to E4M3 (sofie_cuda_quantize_e4m3_f32)", lambda: ops.quantize_e4m3(x, 0.01), 5 * n),
        ("NCHW -> NHWC (sofie_cuda_nchw_to_nhwc)", lambda: ops.nchw_to_nhwc(img), 8 * n),
    ]
    out = []
    for title, call, nbytes in cases:
        try:
            call()
            torch.cuda.synchronize()
            times = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                call()
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            ms = float(np.median(times))
            out.append(dict(kernel=title, bytes=int(nbytes), ms=round(ms, 4), gbs=round(nbytes / (ms * 1e-3) / 1e9, 1),
                            frac=round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)))
        except Exception as e:  # a kernel that refuses a shape must not take the line with it
            out.append(dict(kernel=title, error=f"{type(e).__name__}: {e}"))
    return out


def side_config(workload, batch, steps, warmup, flush, pk, with_cpu, tag):
    """One entry of per_config / large_batch at one GPU."""
    t0 = time.time()
    me = Measured(workload, batch, 0, 1, 0, tag=tag)
    nothing = me.torch.cuda.synchronize
    dev_ms = me.device_timed(steps, warmup, flush, nothing)
    e2e_ms = me.end_to_end(steps, warmup, nothing)
    e2e_pg_ms = me.end_to_end(max(2, steps // 2), 1, nothing, pageable=True)
    ops = me.operator_times(flush, max(3, min(steps, 10)))
    B = me.shard
    entry = dict(
        workload=f"{workload}: {WORKLOAD_DESC[workload]}" + (f" [batch {B}]" if batch else ""), batch=B, steps=steps,
        value=B * steps / (dev_ms * 1e-3), ms_per_step=dev_ms / steps,
        tflops=me.model.flops_per_sample * B * steps / (dev_ms * 1e-3) / 1e12,
        e2e=B * steps / (e2e_ms * 1e-3), e2e_pageable=B * max(2, steps // 2) / (e2e_pg_ms * 1e-3),
        h2d_bytes_per_step=int(me.x_pinned.numel() * 4), d2h_bytes_per_step=int(me.gen.out_elems * 4),
        roofline={k: v for k, v in roofline_of(workload, ops, B, pk).items() if k in ("kernel", "kernel_ms", "frac", "frac_nominal", "achieved", "peak", "unit", "traffic")},
        layer_ms={o["title"]: round(o["ms"], 5) for o in ops}, gpu_launches_per_step=me.kernel_launches(),
    )
    mem = memory_bound_ops(ops, me.model, pk)
    if mem:
        entry["hbm_kernels"] = mem
    if workload == "C4":
        entry["e2e_note"] = "infer() returns its 65536 x 4096 floats as a std::vector by value: building that 1 GB vector, not the device, bounds e2e"
    if with_cpu:
        entry["cpu_baseline"], entry["parity_checked"] = cpu_baseline(workload, me.x, me.output(), me.scales, budget_s=4.0)
    else:
        entry["parity_checked"] = None
    entry["wall_s"] = round(time.time() - t0, 1)
    me.close()
    return entry


def run(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from sofie_b200 import capi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libSOFIE_cuda has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ.pop("NCCL_DEBUG")  # that level only makes NCCL print its version on stdout, next to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    os.environ["SOFIE_CUDA_DEVICE"] = str(local_rank)  # the emitted Session reads its device from here
    affinity = pin_to_gpu_numa_node(local_rank)
    if not affinity.get("pinned"):
        affinity = place_host_memory_near_gpu(local_rank, affinity)
    capi.load()
    clocks = ClockSampler(local_rank)
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    me = Measured(args.workload, args.batch, rank, world, local_rank)
    dev_ms = me.device_timed(args.steps, args.warmup, flush, barrier, clocks)
    e2e_ms = me.end_to_end(args.steps, args.warmup, barrier, clocks)
    h2d_ms = me.h2d_ms()
    ops = me.operator_times(flush, max(5, min(args.steps, 20)))
    extended = clocks.load(me.gen.run_resident)
    clk = clocks.stop("timed windows" if not extended else
                      "0.4 s of replays of the same step right after the timed region (it was shorter than three samples)")

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
    per_rank = torch.tensor([h2d_ms, e2e_ms / args.steps, dev_ms / args.steps], dtype=torch.float64, device="cuda")
    gathered = [per_rank.clone() for _ in range(world)]
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_gather(gathered, per_rank)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    B = me.total_batch
    roof = roofline_of(args.workload, ops, me.shard, pk)
    line = dict(
        metric="samples/s", value=B * args.steps / (dev_ms * 1e-3), unit="samples/s", n_gpus=world,
        steps=args.steps, warmup=args.warmup, ms_per_step=dev_ms / args.steps, higher_is_better=True,
        scaling="strong", vs_baseline=None, dtype=DTYPE[args.workload], data="synthetic",
        config=dict(workload=f"{args.workload}: {WORKLOAD_DESC[args.workload]}" + (f" [batch {args.batch}]" if args.batch else ""),
                    global_batch=B, batch_per_gpu=me.shard,
                    parallelism=f"batch split into {world} contiguous shard(s), one Session per GPU, weights replicated, no collective",
                    l2="flushed between timed steps (256 MiB memset on the Session's stream, outside the event pairs)",
                    launch="CUDA graph of the emitted Session (Session::RunResident)" + (", emitted with Options::kSingleUpload: every operator once over the whole batch" if me.pipelined else ""),
                    e2e_path="emitted C++ Session::infer(float*) from pinned host memory" + (", input uploaded in parts (four, eight from 128 MB on), the model's leading operators launched per part as it arrives" if me.pipelined else ""),
                    host_affinity=affinity),
        tflops=me.model.flops_per_sample * B * args.steps / (dev_ms * 1e-3) / 1e12,
        e2e=dict(value=B * args.steps / (e2e_ms * 1e-3), unit="samples/s",
                 h2d_bytes_per_step=int(me.x_pinned.numel() * 4) * world, d2h_bytes_per_step=int(me.gen.out_elems * 4) * world,
                 per_rank=dict(h2d_copy_alone_ms=[round(float(g[0]), 4) for g in gathered], e2e_ms_per_step=[round(float(g[1]), 4) for g in gathered],
                               device_ms_per_step=[round(float(g[2]), 4) for g in gathered])),
        gpu_launches=me.kernel_launches() * args.steps * world,
        roofline=roof, layer_ms={o["title"]: round(o["ms"], 5) for o in ops}, clocks=clk,
    )
    mem = memory_bound_ops(ops, me.model, pk)
    if mem:
        line["hbm_kernels"] = mem
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            line["cpu_baseline"], line["parity_checked"] = cpu_baseline(args.workload, me.x, me.output(), me.scales)
        me.close()
        del me
        torch.cuda.empty_cache()
        if not args.no_per_config and not args.batch:
            k = max(3, min(args.steps, 10))
            line["per_config"], line["large_batch"] = {}, {}
            for w in ("C1", "C2", "C3", "C4", "C5"):
                if w == args.workload:
                    line["per_config"][w] = dict(see="the headline fields of this line")
                    continue
                try:
                    line["per_config"][w] = side_config(w, None, k if w != "C4" else 3, 3, flush, pk, not args.no_cpu_baseline, "")
                except Exception as e:  # one configuration failing must not take the headline with it
                    line["per_config"][w] = dict(error=f"{type(e).__name__}: {e}")
            for w, b in (("C1", 1 << 18), ("C3", 1 << 18), ("C2", 8192)):
                try:
                    line["large_batch"][f"{w}@{b}"] = side_config(w, b, 5, 3, flush, pk, False, "_large")
                except Exception as e:
                    line["large_batch"][f"{w}@{b}"] = dict(error=f"{type(e).__name__}: {e}")
        if (not args.no_per_config and not args.batch) or args.hbm_ops:
            torch.cuda.empty_cache()
            line["hbm_ops"] = dict(peak_gbs=pk["hbm_gbs"], peak_basis=f"{pk['source']} copy bandwidth", ops=standalone_hbm_ops(torch, pk))
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C5", choices=sorted(WORKLOAD_DESC))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--hbm-ops", action="store_true", help="also time the stand-alone memory-bound operators (always on in the default run)")
    ap.add_argument("--no-per-config", action="store_true", help="only the headline workload (the other configurations are skipped)")
    ap.add_argument("--batch", type=int, default=None, help="another batch / row count than the configuration's (large-batch runs, ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    try:
        if args.impl == "reference":
            return reference_arm(args, rank, world)
        return run(args, rank, world, local_rank)
    except BaseException as e:
        if isinstance(e, SystemExit) and not e.code:
            raise
        # a failing rank says why on its own stderr (the launcher only reports exit codes)
        sys.stderr.write(f"[bench rank {rank}/{world}] {type(e).__name__}: {e}\n{traceback.format_exc()}\n")
        sys.stderr.flush()
        raise


if __name__ == "__main__":
    sys.exit(main())
