#!/usr/bin/env python
"""Benchmark of the B200 backend's hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (N = 1): fp32 GEMM with fused epilogue D = max(0, 1.5 A.B + 0.5 C + bias[col]),
M = N = K = 8192, row-major float32, seeded uniform inputs, in 3xTF32 mode (the
fp32-grade mode).  One step = one call of the operator: two operand-preparation
kernels plus the tcgen05 kernel.  All four matrices are 256 MiB, larger than the
126 MB L2, so no flush is needed between steps.  At N > 1 every rank owns an
8192-row block of A/C/D (weak scaling), B is replicated with an NCCL broadcast
before the timed region, and there is no collective inside it.

The JSON line also carries the TF32-mode figure and the fused-map chain
(a = b + 3c ; d = a*a + b over 2^28 floats) with their own rooflines.

`--impl reference` times the CPU restatement of the reference's Native backend
(oracle/native_oracle.c, the naive matrix_mul kernel with the same epilogue) on
the host cores, on a bounded row slab of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
SEED = 20260101
MAP_N = 1 << 28
METRIC = "fp32_gemm_fused_epilogue_8192cubed"
WORKLOAD = "gemm M=N=K=8192 fp32, D=max(0,1.5*A.B+0.5*C+bias[col]), 3xTF32 split accumulation"


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """SM clock, power and clock-event reasons sampled while the GPU is under the benchmark's load: NVML queries
    from a thread of this process every 5 ms, or, where NVML cannot be loaded, nvidia-smi every 20 ms (started
    early because it needs a moment to come up).  stop() ends the sampling; summary(t0, t1) reports the samples
    taken inside one loaded window."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index
        self.samples = []          # (unix time, sm MHz, power W, [reasons])
        self.max_mhz = None
        self.source = None
        self._thread = None

    def _nvml_loop(self):
        import pynvml as nv
        reasons_of = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                      nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                      nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                      nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
        while not self._stop.is_set():
            try:
                c = nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                pw = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                self.samples.append((time.time(), float(c), pw, [name for bit, name in reasons_of.items() if mask & bit]))
            except Exception:  # a failed read drops one sample, nothing else
                pass
            self._stop.wait(0.005)

    def _start_nvml(self, uuid) -> bool:
        """Reads clocks, power and event reasons through NVML in a thread of this process (read-only queries)."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            self._handle = (nv.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode()) if uuid
                            else nv.nvmlDeviceGetHandleByIndex(self.gpu_index))
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self._handle, nv.NVML_CLOCK_SM))
            nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)
        except Exception:
            return False
        import threading
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._nvml_loop, daemon=True)
        self._thread.start()
        self.source = "nvml, 5 ms period"
        return True

    def start(self, uuid=None):
        if self._start_nvml(uuid):
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi, 20 ms period"
        except OSError:
            self.proc = None

    def stop(self) -> None:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            return
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                c, m, pw = float(f[2]), float(f[3]), float(f[4])
            except ValueError:
                continue
            self.max_mhz = max(self.max_mhz or 0.0, m)
            self.samples.append((ts, c, pw, [n for n, v in zip(self.NAMES, f[5:9]) if v.lower().startswith("active")]))

    def summary(self, t0: float, t1: float) -> dict:
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source (NVML and nvidia-smi unavailable)"]}
        inside = [x for x in self.samples if t0 <= x[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz,
                    "reasons": [f"no samples inside the loaded window ({len(self.samples)} outside)"]}
        return {"sm_mhz": statistics.median(x[1] for x in inside), "sm_min_mhz": min(x[1] for x in inside),
                "sm_max_mhz": self.max_mhz, "reasons": sorted({r for x in inside for r in x[3]}), "samples": len(inside),
                "power_w_max": max(x[2] for x in inside), "source": self.source, "window_s": round(t1 - t0, 3)}


# --------------------------------------------------------------------------- reference arm
def oracle_lib():
    from tests import oracle_lib as O  # the checker doubles as the timed CPU baseline
    return O


def cpu_slab_rate(workers: int, target_s: float):
    """Times the Native-semantics naive kernel with the fused epilogue on the first
    `rows` rows of the 8192^3 problem; returns (tflops, seconds, rows)."""
    import numpy as np
    O = oracle_lib()
    lib = O.load()
    a = O.fill(64 * K, SEED, 1)          # rows of A that the slab can touch (<= 64)
    b = O.fill(K * N, SEED, 2)
    c = O.fill(64 * N, SEED, 3)
    bias = O.fill(N, SEED, 4, kind=1)
    out = np.empty(64 * N, dtype=np.float32)

    def run(ids: int) -> float:
        t0 = time.perf_counter()
        lib.so_par_matmul_naive(a, b, out, 64, N, K, 0, ids, 1.5, 0.5, c.ctypes.data_as(C.c_void_p),
                                bias.ctypes.data_as(C.c_void_p), 1, 1, workers)
        return time.perf_counter() - t0

    calib_ids = 256 * workers
    t = run(calib_ids)
    ids = int(min(64 * N, max(calib_ids, calib_ids * target_s / max(t, 1e-6))))
    ids = max(256, ids // 256 * 256)
    return (lambda: run(ids)), ids


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    workers = max(1, (os.cpu_count() or 2) - 1)
    step, ids = cpu_slab_rate(workers, target_s=2.0)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    flops = 2.0 * K * ids * args.steps
    value = flops / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64 accumulate, f32 store", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "inputs larger than any cache"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": workers, "kind": "port",
                         "sample": f"first {ids} output elements ({ids / N:.2f} rows) of the 8192^3 problem per step; "
                                   "C restatement of Sarek Native (no OCaml toolchain here), faster than the real OCaml "
                                   "backend because it has none of its per-element boxing"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- B200 arm
def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from spoc_b200 import Backend, _lib as L
    from spoc_b200.build import build_library
    from spoc_b200.plugin import _check

    if not os.path.exists(L.LIB_PATH):
        build_library()
    lib = L.load()  # raises when the CUDA library is missing: there is no fallback
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = Backend()
    backend.Device.init()
    dev = backend.Device.get(local_rank)
    backend.Device.set_current(dev)
    tdev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start(getattr(torch.cuda.get_device_properties(local_rank), "uuid", None))  # windowed later

    def fill(t, sid, kind, first=0):
        _check(lib.sb200_fill_f32(dev.id, stream, t.data_ptr(), t.numel(), SEED, sid, kind, 1.0, first))

    A = torch.empty(M * K, dtype=torch.float32, device=tdev)
    B = torch.empty(K * N, dtype=torch.float32, device=tdev)
    Cm = torch.empty(M * N, dtype=torch.float32, device=tdev)
    D = torch.empty(M * N, dtype=torch.float32, device=tdev)
    bias = torch.empty(N, dtype=torch.float32, device=tdev)
    from spoc_b200.sharding import row_block
    first_row, rows = row_block(M * world, world, rank)   # weak scaling: the global problem has M*world rows
    assert rows == M
    fill(A, 1, 0, first=first_row * K)   # this rank's row block of the global A and C
    fill(Cm, 3, 0, first=first_row * N)
    fill(bias, 4, 1)
    bcast_ms = None
    if world > 1:
        if rank == 0:
            fill(B, 2, 0)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(B, src=0)          # B replicated over NVLink into each GPU's own HBM
        e1.record()
        torch.cuda.synchronize()
        bcast_ms = e0.elapsed_time(e1)
    else:
        fill(B, 2, 0)
    torch.cuda.synchronize()

    def gemm(mode):
        _check(lib.sb200_gemm_f32(dev.id, stream, mode, M, N, K, A.data_ptr(), K, B.data_ptr(), N, D.data_ptr(), N,
                                  1.5, Cm.data_ptr(), N, 0.5, bias.data_ptr(), L.ACT_RELU))

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=tdev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warmup, profile=False):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        barrier()
        if profile:
            backend.profile_gemm_read(dev)
            backend.enable_profiling()
        l0 = backend.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        launches = backend.launch_count() - l0
        prof = None
        if profile:
            backend.disable_profiling()
            prof = backend.profile_gemm_read(dev)
        return max_over_ranks(e0.elapsed_time(e1)), launches, prof

    flops_step = 2.0 * M * N * K
    # ---- headline: 3xTF32 ------------------------------------------------------------
    # Two passes of the same timed loop.  The first starts on a GPU that was idle a moment ago and is over
    # before the power management has settled ("burst").  Then the same step runs untimed for --preload-s
    # seconds, and the second pass — the headline — runs at the clock the 1 kW cap sustains, with enough
    # load behind it for the clock and reason samples to describe the timed steps.
    burst = None
    if args.preload_s > 0:
        t_b0 = time.time()
        ms_b, _, prof_b = timed(lambda: gemm(L.MODE_3XTF32), args.steps, args.warmup, profile=True)
        t_b1 = time.time()
        burst = {"value": world * flops_step / (ms_b / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                 "ms_per_step": ms_b / args.steps, "kernel_ms": prof_b["main_ms"] / max(prof_b["calls"], 1),
                 "note": "same loop, run first on an idle GPU, before the clocks settle under the power cap"}
    t_pre = time.time()
    while time.time() - t_pre < args.preload_s:
        for _ in range(5):
            gemm(L.MODE_3XTF32)
        torch.cuda.synchronize()
    t_w0 = time.time()
    ms, launches, prof = timed(lambda: gemm(L.MODE_3XTF32), args.steps, args.warmup, profile=True)
    t_w1 = time.time()
    _check(lib.sb200_device_synchronize(dev.id))  # also surfaces a device-side timeout flag
    ms_step = ms / args.steps
    value = world * flops_step / (ms_step * 1e-3) / 1e12
    sustained = args.preload_s >= 0.25
    burst_peak = peaks["bf16_tflops"] / 2.0
    tf32_peak = peaks["bf16_tflops_sustained"] / 2.0 if sustained else burst_peak
    main_ms = prof["main_ms"] / max(prof["calls"], 1)
    prep_ms = prof["prep_ms"] / max(prof["calls"], 1)
    achieved = flops_step / (main_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "gemm_pair_kernel<3, true>", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
        "frac": achieved / tf32_peak,
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this size, taken from an
        # ncu capture of this same kernel and size (a profiler figure, not measured in this run)
        "traffic": 8.144e9 + 0.262e9, "traffic_unit": "bytes per launch (ncu capture of this kernel at this size)",
        "peak_source": (f"{peaks['source']}: bf16 sustained {peaks['bf16_tflops_sustained']} TF/s / 2 = dense TF32 under the power cap "
                        "(the timed steps follow a pre-load)" if sustained else
                        f"{peaks['source']}: bf16 burst {peaks['bf16_tflops']} TF/s / 2 = dense TF32"),
        "frac_of_burst_peak": achieved / burst_peak,
        "mma_frac": 3.0 * achieved / tf32_peak,
        "kernel_ms": main_ms, "prep_ms": prep_ms,
        "note": "achieved counts the algorithmic 2*M*N*K flops; 3xTF32 issues 3 MMAs per k-step, mma_frac is the tensor-pipe share",
    }

    # ---- TF32 mode ----------------------------------------------------------------------
    s2 = max(3, min(args.steps, 10))
    t_t0 = time.time()
    ms2, _, prof2 = timed(lambda: gemm(L.MODE_TF32), s2, 3, profile=True)   # straight after the headline pass: same regime
    t_t1 = time.time()
    main2 = prof2["main_ms"] / max(prof2["calls"], 1)
    tf32_mode = {
        "value": world * flops_step / (ms2 / s2 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms2 / s2,
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<1, true> (operands read directly, no preparation)", "achieved": flops_step / (main2 * 1e-3) / 1e12,
                     "peak": tf32_peak, "unit": "TFLOP/s", "frac": flops_step / (main2 * 1e-3) / 1e12 / tf32_peak,
                     "peak_source": roofline["peak_source"],
                     "frac_of_burst_peak": flops_step / (main2 * 1e-3) / 1e12 / burst_peak,
                     "kernel_ms": main2, "prep_ms": prof2["prep_ms"] / max(prof2["calls"], 1)},
    }
    clocks = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(t_w0, t_w1)
        tf32_mode["clocks"] = sampler.summary(t_t0, t_t1)
        if burst is not None:
            burst["clocks"] = sampler.summary(t_b0, t_b1)

    # ---- e2e: host buffers, copies inside the timed region ---------------------------------
    hA = torch.empty(M * K, dtype=torch.float32).pin_memory()
    hB = torch.empty(K * N, dtype=torch.float32).pin_memory()
    hC = torch.empty(M * N, dtype=torch.float32).pin_memory()
    hbias = torch.empty(N, dtype=torch.float32).pin_memory()
    hD = torch.empty(M * N, dtype=torch.float32).pin_memory()
    for h, d in ((hA, A), (hB, B), (hC, Cm), (hbias, bias)):
        h.copy_(d)
    torch.cuda.synchronize()

    def e2e_step():
        # the call a user with host data makes: one C-ABI call, copies inside it
        _check(lib.sb200_gemm_f32_host(dev.id, L.MODE_3XTF32, M, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N,
                                       1.5, hC.data_ptr(), N, 0.5, hbias.data_ptr(), L.ACT_RELU))

    s3 = max(3, min(args.steps, 10))
    ms3, _, _ = timed(e2e_step, s3, 2)
    e2e = {"value": world * flops_step / (ms3 / s3 * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 4 * (M * K + K * N + M * N + N), "d2h_bytes_per_step": 4 * M * N,
           "ms_per_step": ms3 / s3,
           "api": "sb200_gemm_f32_host: pinned host A, B, C, bias in, D out; copies, row-block GEMMs and copy-out overlapped"}
    # the same call on ordinary pageable host memory (what a Bigarray is): staged by host threads inside the call
    pA, pB, pC, pD = (torch.empty(n, dtype=torch.float32) for n in (M * K, K * N, M * N, M * N))
    pA.copy_(hA); pB.copy_(hB); pC.copy_(hC)

    def e2e_pageable_step():
        _check(lib.sb200_gemm_f32_host(dev.id, L.MODE_3XTF32, M, N, K, pA.data_ptr(), K, pB.data_ptr(), N, pD.data_ptr(), N,
                                       1.5, pC.data_ptr(), N, 0.5, hbias.data_ptr(), L.ACT_RELU))

    ms5, _, _ = timed(e2e_pageable_step, 3, 1)
    e2e["pageable_host_buffers"] = {"value": world * flops_step / (ms5 / 3 * 1e-3) / 1e12, "unit": "TFLOP/s",
                                    "ms_per_step": ms5 / 3}
    # the plugin path itself: Execute.run_vectors on the epilogue kernel's IR with host-resident vectors, i.e.
    # Transfer.to_device of every argument, the launch, Transfer.to_cpu of the result, one after the other
    from spoc_b200 import Vector, run_vectors, dims1d, sarek_ir
    epi_ir = sarek_ir.matmul_naive_ir(epilogue=dict(alpha=1.5, beta=0.5, c="c", bias="bias", relu=True))
    vecs = [Vector(backend, t.numpy()) for t in (pA, pB, pC)] + [Vector(backend, hbias.numpy().copy()), Vector(backend, pD.numpy())]

    def plugin_step():
        for v in vecs[:4]:
            v.location = Vector.CPU          # the host copy is the valid one again: the next launch re-uploads it
        run_vectors(backend, device=dev, ir=epi_ir, args=vecs + [("int32", M), ("int32", N), ("int32", K)],
                    block=dims1d(256), grid=dims1d((M * N + 255) // 256))
        vecs[4].to_array()

    ms6, _, _ = timed(plugin_step, 3, 1)
    e2e["plugin_run_vectors"] = {"value": world * flops_step / (ms6 / 3 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms6 / 3,
                                 "note": "run_vectors on the kernel's IR, pageable host vectors, synchronous transfers as in the reference"}
    for v in vecs:
        v.free()
    del hA, hB, hC, hD, pA, pB, pC, pD

    # ---- fused-map chain (HBM bound) ---------------------------------------------------------
    fused_map = None
    if world == 1:
        del A, Cm
        b = torch.empty(MAP_N, dtype=torch.float32, device=tdev)
        c = torch.empty(MAP_N, dtype=torch.float32, device=tdev)
        d = torch.empty(MAP_N, dtype=torch.float32, device=tdev)
        fill(b, 2, 0)
        fill(c, 3, 0)
        s4 = max(5, min(args.steps, 20))
        ms4, l4, _ = timed(lambda: _check(lib.sb200_chain_triad_square_f32(dev.id, stream, d.data_ptr(), 0, b.data_ptr(),
                                                                         c.data_ptr(), 3.0, MAP_N)), s4, 3)
        gbs = 12.0 * MAP_N / (ms4 / s4 * 1e-3) / 1e9
        fused_map = {"workload": "a=b+3c; d=a*a+b fused, N=2^28 float32, intermediate eliminated", "value": gbs,
                     "unit": "GB/s", "ms_per_step": ms4 / s4, "launches_per_step": l4 / s4,
                     "roofline": {"bound": "hbm", "kernel": "map2_vec_kernel<ChainOp>", "achieved": gbs,
                                  "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                  # ncu capture at 2^26 elements scaled x4 (traffic is proportional to N: no reuse)
                                  "traffic": 4 * (536.9e6 + 268.4e6),
                                  "traffic_unit": "bytes per launch (ncu capture at 2^26 elements, scaled x4)",
                                  "peak_source": f"{peaks['source']} copy bandwidth",
                                  "frac_of_nominal_8TBs": gbs / 8000.0}}

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        workers = max(1, (os.cpu_count() or 2) - 1)
        step, ids = cpu_slab_rate(workers, target_s=12.0)
        dt = step()
        cpu_baseline = {"value": 2.0 * K * ids / dt / 1e12, "unit": "TFLOP/s", "cores": workers, "kind": "port",
                        "sample": f"first {ids} output elements ({ids / N:.2f} rows) of the same 8192^3 problem, "
                                  f"{dt:.1f} s; C restatement of Sarek Native's naive kernel with the epilogue"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3 (f32 in/out)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": M, "l2": "inputs larger than L2 (4 x 256 MiB per GPU)", "preload_s": args.preload_s,
                       "sharding": "row blocks of A/C/D per rank, B replicated by NCCL broadcast before the timed region"},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "burst": burst, "tf32_mode": tf32_mode, "fused_map": fused_map, "b_broadcast_ms": bcast_ms,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_transfer_case(lib, dev, S: int) -> None:
    """Whole-vector copies of S*S float32 (1 GiB at --size 16384) between the device and (a) pageable host
    memory through the library's staged path, (b) the same with the staged path switched off in a child
    process, (c) pinned host memory.  Wall-clock of the synchronous call, best of 3."""
    import ctypes as Ct
    import numpy as np
    from spoc_b200.plugin import _check
    n = S * S
    dptr = Ct.c_uint64(0)
    _check(lib.sb200_mem_alloc(dev.id, 4 * n, Ct.byref(dptr)))
    host = np.ones(n, np.float32)
    pinned = Ct.c_void_p()
    _check(lib.sb200_host_alloc(4 * n, Ct.byref(pinned)))

    def best(fn):
        fn()
        ts = []
        for _ in range(3):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return 4 * n / min(ts) / 1e9

    out = {"case": "transfer", "bytes": 4 * n, "unit": "GB/s",
           "staged_path": os.environ.get("SAREK_B200_STAGED_COPY", "1") != "0",
           "pageable_htod": best(lambda: _check(lib.sb200_memcpy_htod(dev.id, dptr.value, host.ctypes.data, 4 * n))),
           "pageable_dtoh": best(lambda: _check(lib.sb200_memcpy_dtoh(dev.id, host.ctypes.data, dptr.value, 4 * n))),
           "pinned_htod": best(lambda: _check(lib.sb200_memcpy_htod(dev.id, dptr.value, pinned, 4 * n))),
           "pinned_dtoh": best(lambda: _check(lib.sb200_memcpy_dtoh(dev.id, pinned, dptr.value, 4 * n)))}
    _check(lib.sb200_host_free(pinned))
    _check(lib.sb200_mem_free(dev.id, dptr.value))
    print(json.dumps(out), flush=True)


def run_tiles_case(lib, dev) -> None:
    """Per-call time of sb200_gemm_f32 (plain product, aligned operands) for the tile widths of the CTA-pair kernel
    — 256, 128, 64 columns and the automatic choice — over a range of sizes and both modes: 5 warm-up calls, then
    back-to-back calls and one synchronise, wall-clock / calls (launch gaps included)."""
    import numpy as np
    from spoc_b200 import Backend, _lib as L
    from spoc_b200.plugin import _check
    b = Backend()
    shapes = [(128, 128, 128), (256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (1280, 1280, 1280),
              (1536, 1536, 1536), (1792, 1792, 1792), (2048, 2048, 2048), (2560, 2560, 2560), (4096, 4096, 4096),
              (512, 4096, 512), (4096, 512, 4096), (1024, 1024, 8192), (64, 8192, 8192), (8192, 4096, 4096)]
    rows = []
    for (M, N, K) in shapes:
        A, B, D = (b.Memory.alloc(dev, n, np.float32) for n in (M * K, K * N, M * N))
        _check(lib.sb200_fill_f32(dev.id, 0, A.ptr, M * K, SEED, 1, 0, 1.0, 0))
        _check(lib.sb200_fill_f32(dev.id, 0, B.ptr, K * N, SEED, 2, 0, 1.0, 0))
        for mode, label in ((L.MODE_TF32, "tf32"), (L.MODE_3XTF32, "3xtf32")):
            row = {"M": M, "N": N, "K": K, "mode": label}
            for tile in (256, 128, 64, 0):
                _check(lib.sb200_set_gemm_tile_n(tile))
                call = lambda: _check(lib.sb200_gemm_f32(dev.id, 0, mode, M, N, K, A.ptr, K, B.ptr, N, D.ptr, N, 1.0, 0, 0, 0.0, 0, 0))
                for _ in range(5):
                    call()
                _check(lib.sb200_device_synchronize(dev.id))
                calls = 200 if M * N * K < 2 ** 33 else 30
                t0 = time.perf_counter()
                for _ in range(calls):
                    call()
                _check(lib.sb200_device_synchronize(dev.id))
                row["auto_us" if tile == 0 else f"tile{tile}_us"] = round((time.perf_counter() - t0) / calls * 1e6, 1)
            row["auto_tflops"] = round(2.0 * M * N * K / row["auto_us"] / 1e6, 1)
            rows.append(row)
        for m in (A, B, D):
            b.Memory.free(m)
    _check(lib.sb200_set_gemm_tile_n(0))
    print(json.dumps({"case": "tiles", "unit": "us per call", "rows": rows}), flush=True)


def run_case(args) -> None:
    """A small single-operator run for profiler captures: one warm-up call and two
    measured calls of one operator on inputs larger than L2 but well under a GB."""
    import torch

    from spoc_b200 import Backend, _lib as L
    from spoc_b200.plugin import _check
    lib = L.load()
    backend = Backend()
    backend.Device.init()
    dev = backend.Device.get(0)
    backend.Device.set_current(dev)
    torch.cuda.set_device(0)
    tdev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream
    S = args.size
    if args.case == "transfer":
        return run_transfer_case(lib, dev, S)
    if args.case == "tiles":
        return run_tiles_case(lib, dev)
    if args.case in ("gemm3", "gemm1"):
        mode = L.MODE_3XTF32 if args.case == "gemm3" else L.MODE_TF32
        bufs = [torch.empty(S * S, dtype=torch.float32, device=tdev) for _ in range(4)]
        bias = torch.empty(S, dtype=torch.float32, device=tdev)
        for i, t in enumerate(bufs[:3]):
            _check(lib.sb200_fill_f32(dev.id, stream, t.data_ptr(), t.numel(), SEED, i + 1, 0, 1.0, 0))
        _check(lib.sb200_fill_f32(dev.id, stream, bias.data_ptr(), S, SEED, 4, 1, 1.0, 0))
        fn = lambda: _check(lib.sb200_gemm_f32(dev.id, stream, mode, S, S, S, bufs[0].data_ptr(), S, bufs[1].data_ptr(), S,
                                               bufs[3].data_ptr(), S, 1.5, bufs[2].data_ptr(), S, 0.5, bias.data_ptr(), 1))
        work, unit = 2.0 * S ** 3 / 1e12, "TFLOP/s"
    else:
        n = S * S
        bufs = [torch.empty(n, dtype=torch.float32, device=tdev) for _ in range(3)]
        for i, t in enumerate(bufs[:2]):
            _check(lib.sb200_fill_f32(dev.id, stream, t.data_ptr(), n, SEED, i + 2, 0, 1.0, 0))
        fn = lambda: _check(lib.sb200_chain_triad_square_f32(dev.id, stream, bufs[2].data_ptr(), 0, bufs[0].data_ptr(),
                                                             bufs[1].data_ptr(), 3.0, n))
        work, unit = 12.0 * n / 1e9, "GB/s"
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    fn()
    e1.record()
    torch.cuda.synchronize()
    _check(lib.sb200_device_synchronize(dev.id))
    ms = e0.elapsed_time(e1) / 2
    print(json.dumps({"case": args.case, "size": S, "ms_per_call": ms, "rate": work / (ms * 1e-3), "unit": unit}), flush=True)


def run_gather(args, rank: int, local_rank: int, world: int) -> None:
    """Strong-scaling run of the large square GEMM with epilogue and a gathered result: M = N = K = --size
    (default 32768), rows of A/C/D split over the ranks, B replicated.  Two ways to leave the whole D on every
    GPU are timed: the GEMM followed by an NCCL all-gather of the row blocks, and the GEMM whose epilogue stores
    each tile into every GPU's copy (peer stores over NVLink)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from spoc_b200 import Backend, _lib as L
    from spoc_b200.plugin import _check
    from spoc_b200.sharding import row_block
    lib = L.load()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = Backend()
    backend.Device.init()
    dev = backend.Device.get(local_rank)
    backend.Device.set_current(dev)
    tdev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    S = args.size
    r0, rows = row_block(S, world, rank)

    def fill(ptr, n, sid, kind, first=0):
        _check(lib.sb200_fill_f32(dev.id, stream, ptr, n, SEED, sid, kind, 1.0, first))

    A = torch.empty(rows * S, dtype=torch.float32, device=tdev)
    Cm = torch.empty(rows * S, dtype=torch.float32, device=tdev)
    B = torch.empty(S * S, dtype=torch.float32, device=tdev)
    bias = torch.empty(S, dtype=torch.float32, device=tdev)
    fill(A.data_ptr(), A.numel(), 1, 0, r0 * S)
    fill(Cm.data_ptr(), Cm.numel(), 3, 0, r0 * S)
    fill(bias.data_ptr(), S, 4, 1)
    if rank == 0:
        fill(B.data_ptr(), B.numel(), 2, 0)
    if world > 1:
        dist.broadcast(B, src=0)
    D_nccl = torch.empty(S * S, dtype=torch.float32, device=tdev)     # gathered by NCCL
    D_own = backend.Memory.alloc(dev, S * S, np.float32)              # gathered by the epilogue (IPC-shareable memory)
    copies = [D_own.ptr]
    opened = []
    if world > 1:
        handle = C.create_string_buffer(64)
        _check(lib.sb200_ipc_export(dev.id, D_own.ptr, handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        for r in range(world):
            if r != rank:
                pp = C.c_uint64(0)
                _check(lib.sb200_ipc_open(dev.id, C.create_string_buffer(handles[r], 64), C.byref(pp)))
                copies.append(pp.value)
                opened.append(pp.value)
    ptrs = (C.c_uint64 * len(copies))(*copies)
    torch.cuda.synchronize()

    def step_nccl():
        shard = D_nccl[r0 * S:(r0 + rows) * S]
        _check(lib.sb200_gemm_f32(dev.id, stream, L.MODE_3XTF32, rows, S, S, A.data_ptr(), S, B.data_ptr(), S, shard.data_ptr(), S,
                                  1.5, Cm.data_ptr(), S, 0.5, bias.data_ptr(), L.ACT_RELU))
        if world > 1:
            dist.all_gather_into_tensor(D_nccl, shard)

    def step_fused():
        _check(lib.sb200_gemm_f32_gather(dev.id, stream, L.MODE_3XTF32, rows, S, S, A.data_ptr(), S, B.data_ptr(), S, ptrs,
                                         len(copies), r0, S, 1.5, Cm.data_ptr(), S, 0.5, bias.data_ptr(), L.ACT_RELU))

    def timed(fn):
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1) / args.steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=tdev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    ms_nccl = timed(step_nccl)
    ms_fused = timed(step_fused)
    # the two gathered results must agree bit for bit on this rank
    own = torch.empty(S * S, dtype=torch.float32, device=tdev)
    _check(lib.sb200_memcpy_dtod(dev.id, own.data_ptr(), D_own.ptr, 4 * S * S))
    same = bool(torch.equal(own, D_nccl))
    if world > 1:
        flag = torch.tensor([1 if same else 0], device=tdev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        same = bool(flag.item())
        dist.barrier()
    for pp in opened:
        _check(lib.sb200_ipc_close(dev.id, pp))
    flops = 2.0 * S ** 3
    if rank == 0:
        print(json.dumps({
            "metric": f"fp32_gemm_fused_epilogue_{S}cubed_gathered", "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "scaling": "strong", "higher_is_better": True, "data": "synthetic", "dtype": "tf32x3 (f32 in/out)",
            "config": {"workload": f"gemm M=N=K={S} with epilogue, rows of A/C/D split over the ranks, whole D on every GPU"},
            "value": flops / (ms_fused * 1e-3) / 1e12, "ms_per_step": ms_fused,
            "gemm_then_nccl_all_gather": {"value": flops / (ms_nccl * 1e-3) / 1e12, "ms_per_step": ms_nccl},
            "gather_fused_in_epilogue": {"value": flops / (ms_fused * 1e-3) / 1e12, "ms_per_step": ms_fused},
            "results_identical": same}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_skinny(args, rank: int, local_rank: int, world: int) -> None:
    """Strong-scaling run of the skinny GEMM: C = A.B with M = 65536, N = K = 4096, rows of A drawn from N(0,1),
    B from N(0,1/sqrt(K)); rows of A and C split over the ranks, B broadcast from rank 0 (NCCL).  Timed twice:
    with B already on every GPU, and with the broadcast of B inside every timed step."""
    import math

    import torch
    import torch.distributed as dist

    from spoc_b200 import Backend, _lib as L
    from spoc_b200.plugin import _check
    from spoc_b200.sharding import row_block
    lib = L.load()
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = Backend()
    backend.Device.init()
    dev = backend.Device.get(local_rank)
    backend.Device.set_current(dev)
    tdev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream().cuda_stream
    Mt, Nn, Kk = 65536, 4096, 4096
    r0, rows = row_block(Mt, world, rank)
    A = torch.empty(rows * Kk, dtype=torch.float32, device=tdev)
    Cm = torch.empty(rows * Nn, dtype=torch.float32, device=tdev)
    B = torch.empty(Kk * Nn, dtype=torch.float32, device=tdev)
    _check(lib.sb200_fill_f32(dev.id, stream, A.data_ptr(), A.numel(), SEED, 1, 2, 1.0, r0 * Kk))
    if rank == 0:
        _check(lib.sb200_fill_f32(dev.id, stream, B.data_ptr(), B.numel(), SEED, 2, 2, 1.0 / math.sqrt(Kk), 0))
    if world > 1:
        dist.broadcast(B, src=0)
    torch.cuda.synchronize()
    out = {}
    for mode, label in ((L.MODE_3XTF32, "3xtf32"), (L.MODE_TF32, "tf32")):
        def gemm():
            _check(lib.sb200_gemm_f32(dev.id, stream, mode, rows, Nn, Kk, A.data_ptr(), Kk, B.data_ptr(), Nn, Cm.data_ptr(), Nn,
                                      1.0, 0, 0, 0.0, 0, L.ACT_NONE))

        def gemm_after_broadcast():
            if world > 1:
                dist.broadcast(B, src=0)
            gemm()

        for name, fn in (("b_resident", gemm), ("b_broadcast_timed", gemm_after_broadcast)):
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms = e0.elapsed_time(e1) / args.steps
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device=tdev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            out.setdefault(label, {})[name] = {"ms_per_step": ms, "value": 2.0 * Mt * Nn * Kk / (ms * 1e-3) / 1e12}
    if rank == 0:
        print(json.dumps({
            "metric": "fp32_gemm_65536x4096x4096_row_sharded", "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "scaling": "strong", "higher_is_better": True, "data": "synthetic",
            "dtype": "tf32x3 (f32 in/out)",
            "config": {"workload": "gemm M=65536 N=K=4096, A ~ N(0,1), B ~ N(0,1/sqrt(K)), rows of A/C split over the ranks, "
                                   "B broadcast from rank 0 (64 MiB, NCCL)"},
            "value": out["3xtf32"]["b_resident"]["value"], "ms_per_step": out["3xtf32"]["b_resident"]["ms_per_step"],
            "modes": out}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm8192", choices=["gemm8192", "gather", "skinny"],
                    help="gemm8192: the headline run; gather: large square GEMM with the result gathered on every GPU; "
                         "skinny: 65536x4096x4096 GEMM, rows split over the ranks, B broadcast")
    ap.add_argument("--case", default=None, choices=["gemm3", "gemm1", "map", "transfer", "tiles"],
                    help="profiler-sized single-operator run (square size --size; map uses size^2 elements)")
    ap.add_argument("--size", type=int, default=4096)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--preload-s", type=float, default=0.5,
                    help="seconds of untimed identical steps before the headline pass, so that it is measured at the "
                         "sustained clock; 0 measures the first pass on the idle GPU only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.case:
        run_case(args)
    elif args.workload == "gather":
        if args.size == 4096:
            args.size = 32768
        run_gather(args, rank, local_rank, world)
    elif args.workload == "skinny":
        run_skinny(args, rank, local_rank, world)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
