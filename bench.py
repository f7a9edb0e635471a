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
WORKLOAD = "gemm M=N=K=8192 fp32 in/out, D=max(0,1.5*A.B+0.5*C+bias[col]), seeded uniform inputs (BASELINE configs[2])"
NOMINAL_TF32_TFLOPS = 1100.0   # dense TF32 tensor peak of a B200, nominal
NOMINAL_HBM_GBS = 8000.0


def make_config(args) -> dict:
    """The `config` of the JSON line: the same dict in both arms (what differs between the arms — arithmetic,
    threads, sampling — is said in `dtype`, `cpu_baseline` and `arm`)."""
    return {"workload": WORKLOAD, "rows_per_gpu": M, "l2": "inputs larger than L2 (4 x 256 MiB per GPU)",
            "sharding": "row blocks of A/C/D per GPU, B replicated (NCCL broadcast) before the timed region"}


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
    """The reference's own CPU implementation of the path, timed on this box's host cores: Sarek's Native backend runs
    the kernel on (cores - 1) OCaml domains (sarek/sarek/Sarek_cpu_runtime.ml:1190); with no OCaml toolchain on the
    box the C restatement of that backend (oracle/native_oracle.c, same partition of the global ids over the workers,
    same double arithmetic) is what runs.  Each step computes a bounded slab of output elements of the 8192^3
    problem with the fused epilogue; the full-problem time is extrapolated linearly from it."""
    if rank != 0:
        return
    workers = max(1, (os.cpu_count() or 2) - 1)
    step, ids = cpu_slab_rate(workers, target_s=float(os.environ.get("SAREK_BENCH_TARGET_S", "2.0")))
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    flops = 2.0 * K * ids * args.steps
    value = flops / dt / 1e12
    sample_ms = dt / args.steps * 1e3
    full_ms = sample_ms * (float(M) * N / ids)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": full_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64 accumulate, f32 store", "data": "synthetic",
        "config": make_config(args),
        "arm": {"threads": workers, "sample_ms_per_step": sample_ms, "sample_elements_per_step": ids,
                "note": f"ms_per_step is extrapolated: the time of one full 8192^3 step at the rate measured on a slab of {ids} "
                        f"output elements ({ids / N:.2f} rows) per step on {workers} threads"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": workers, "kind": "port",
                         "sample": f"first {ids} output elements ({ids / N:.2f} rows) of the 8192^3 problem per step, "
                                   f"extrapolated to the full problem; C restatement of Sarek Native (no OCaml toolchain here), "
                                   "faster than the real OCaml backend because it has none of its per-element boxing"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- B200 arm
def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from spoc_b200 import _lib as L
    from spoc_b200.build import build_library
    from spoc_b200.plugin import _check

    if not os.path.exists(L.LIB_PATH):
        build_library()
    L.load()  # raises when the CUDA library is missing: there is no fallback
    ctx = Ctx(rank, local_rank, world)
    lib, backend, dev, tdev, stream = ctx.lib, ctx.backend, ctx.dev, ctx.tdev, ctx.stream
    host_group = dist.new_group(backend="gloo") if world > 1 else None   # host-side barrier: parks ranks without GPU work
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
        "traffic": 4.832e9 + 0.256e9,
        "traffic_unit": "bytes per launch (ncu capture of this kernel at this size with the soft lockstep on, "
                        "profiles/gemm_pair_kernel_4096x32768x32768_ncu.md; 6.63e9 + 0.26e9 with SAREK_B200_LOCKSTEP=0; algorithmic "
                        "bytes 1.28e9: A, B, their low-part panels, C in, D out)",
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
    # ---- the fp16 three-term split: fp32-grade accuracy (same bound as 3xTF32 on these inputs) at the fp16 tensor rate ---
    s5 = max(3, min(args.steps, 10))
    ms_h, _, prof_h = timed(lambda: gemm(L.MODE_3XF16), s5, 3, profile=True)
    main_h = prof_h["main_ms"] / max(prof_h["calls"], 1)
    f16_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    f16_split_mode = {
        "value": world * flops_step / (ms_h / s5 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_h / s5,
        "note": "SB200_MODE_3XF16: operands scaled by powers of two and split hi + lo in fp16, three kind::f16 MMAs per k-step; "
                "parity bound 1e-5*sqrt(K) as for 3xTF32 (tests/test_gpu_gemm.py::test_f16_split_*); not the headline because its "
                "accuracy depends on the dynamic range inside each matrix",
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<4, false> (fp16 panels)", "achieved": flops_step / (main_h * 1e-3) / 1e12,
                     "peak": f16_peak, "unit": "TFLOP/s", "frac": flops_step / (main_h * 1e-3) / 1e12 / f16_peak,
                     "mma_frac": 3.0 * flops_step / (main_h * 1e-3) / 1e12 / f16_peak,
                     "peak_source": f"{peaks['source']}: dense bf16/fp16 library GEMM, {'sustained' if sustained else 'burst'}",
                     "kernel_ms": main_h, "prep_ms": prof_h["prep_ms"] / max(prof_h["calls"], 1)}}
    ms_q, _, prof_q = timed(lambda: gemm(L.MODE_F16), s5, 3, profile=True)
    main_q = prof_q["main_ms"] / max(prof_q["calls"], 1)
    f16_single_mode = {
        "value": world * flops_step / (ms_q / s5 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_q / s5,
        "note": "SB200_MODE_F16: one kind::f16 MMA per k-step on power-of-two-scaled fp16 panels; TF32 mode's 11 significant bits "
                "and error bound (2e-3) at the fp16 tensor rate",
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<2, false> (fp16 panels)", "achieved": flops_step / (main_q * 1e-3) / 1e12,
                     "peak": f16_peak, "unit": "TFLOP/s", "frac": flops_step / (main_q * 1e-3) / 1e12 / f16_peak,
                     "peak_source": f16_split_mode["roofline"]["peak_source"], "kernel_ms": main_q,
                     "prep_ms": prof_q["prep_ms"] / max(prof_q["calls"], 1)}}
    # ---- the mixed mode: 3xTF32's three terms with the two cross terms on the fp16 pipe ---------------------------
    ms_x, _, prof_x = timed(lambda: gemm(L.MODE_3XMIXED), s5, 3, profile=True)
    main_x = prof_x["main_ms"] / max(prof_x["calls"], 1)
    mixed_mode = {
        "value": world * flops_step / (ms_x / s5 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_x / s5,
        "note": "SB200_MODE_3XMIXED: hi*hi as TF32 MMAs on the caller's fp32 matrices, hi*lo + lo*hi as fp16 MMAs on panels "
                "with one power-of-two scale per matrix, the accumulated cross terms rescaled inside the tensor core "
                "(scale-input-d); the error of 3xTF32 for elements within 2^29 of their matrix's largest "
                "(tests/test_gpu_gemm_mixed.py); kernel_ms covers the mixed kernel and the two gated 3xTF32 launches behind it",
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel<5, true>", "achieved": flops_step / (main_x * 1e-3) / 1e12,
                     "peak": tf32_peak, "unit": "TFLOP/s", "frac": flops_step / (main_x * 1e-3) / 1e12 / tf32_peak,
                     "mma_frac": 2.0 * flops_step / (main_x * 1e-3) / 1e12 / tf32_peak,
                     "peak_source": roofline["peak_source"], "kernel_ms": main_x,
                     "prep_ms": prof_x["prep_ms"] / max(prof_x["calls"], 1)}}
    clocks = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(t_w0, t_w1)
        tf32_mode["clocks"] = sampler.summary(t_t0, t_t1)
        if burst is not None:
            burst["clocks"] = sampler.summary(t_b0, t_b1)

    # ---- e2e: host buffers, copies inside the timed region ---------------------------------
    # One GPU: the headline is the plugin path itself — Execute.run_vectors on the epilogue kernel's IR with host-resident
    # vectors in ordinary pageable memory (what a Bigarray is): the uploads of Transfer.to_device folded into the launch
    # call, which overlaps them with the GEMM by row blocks, then Transfer.to_cpu of the result.  The direct operator on pinned and on
    # pageable buffers (one C-ABI call that overlaps copies and row-block GEMMs) is reported beside it.
    # Several GPUs: the call a single-process host makes, sb200_gemm_sharded_host on a group of all the GPUs — B
    # crosses PCIe once (a band of rows per GPU, all-gathered over NVLink), every GPU moves only its own rows — issued by
    # rank 0 on pageable operands of world x 8192 rows while the other ranks wait at a host-side barrier with
    # nothing running on their GPUs.
    e2e = None
    e2e_bytes_in, e2e_bytes_out = 4 * (M * K + K * N + M * N + N), 4 * M * N
    if world == 1:
        hA = torch.empty(M * K, dtype=torch.float32).pin_memory()
        hB = torch.empty(K * N, dtype=torch.float32).pin_memory()
        hC = torch.empty(M * N, dtype=torch.float32).pin_memory()
        hbias = torch.empty(N, dtype=torch.float32).pin_memory()
        hD = torch.empty(M * N, dtype=torch.float32).pin_memory()
        for h, d in ((hA, A), (hB, B), (hC, Cm), (hbias, bias)):
            h.copy_(d)
        torch.cuda.synchronize()

        def e2e_pinned_step():
            _check(lib.sb200_gemm_f32_host(dev.id, L.MODE_3XTF32, M, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N,
                                           1.5, hC.data_ptr(), N, 0.5, hbias.data_ptr(), L.ACT_RELU))

        s3 = max(3, min(args.steps, 10))
        ms3, _, _ = timed(e2e_pinned_step, s3, 2)
        pA, pB, pC, pD = (torch.empty(n, dtype=torch.float32) for n in (M * K, K * N, M * N, M * N))
        pA.copy_(hA); pB.copy_(hB); pC.copy_(hC)

        def e2e_pageable_step():
            _check(lib.sb200_gemm_f32_host(dev.id, L.MODE_3XTF32, M, N, K, pA.data_ptr(), K, pB.data_ptr(), N, pD.data_ptr(), N,
                                           1.5, pC.data_ptr(), N, 0.5, hbias.data_ptr(), L.ACT_RELU))

        ms5, _, _ = timed(e2e_pageable_step, 3, 1)
        from spoc_b200 import Vector, run_vectors, dims1d, sarek_ir
        epi_ir = sarek_ir.matmul_naive_ir(epilogue=dict(alpha=1.5, beta=0.5, c="c", bias="bias", relu=True))
        vecs = [Vector(backend, t.numpy()) for t in (pA, pB, pC)] + [Vector(backend, hbias.numpy().copy()), Vector(backend, pD.numpy())]

        def plugin_step():
            for v in vecs[:4]:
                v.location = Vector.CPU          # the host copy is the valid one again: the next launch re-uploads it
            run_vectors(backend, device=dev, ir=epi_ir, args=vecs + [("int32", M), ("int32", N), ("int32", K)],
                        block=dims1d(256), grid=dims1d((M * N + 255) // 256))
            vecs[4].to_array()

        s6 = max(3, min(args.steps, 5))
        ms6, _, _ = timed(plugin_step, s6, 3)   # the plugin pins a vector's host array in place on its second transfer: in the warm-up
        e2e = {"value": flops_step / (ms6 / s6 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms6 / s6,
               "h2d_bytes_per_step": e2e_bytes_in, "d2h_bytes_per_step": e2e_bytes_out,
               "api": "Execute.run_vectors mirror (spoc_b200.plugin.run_vectors) on the epilogue kernel's IR: host vectors in "
                      "ordinary (pageable) memory, which the plugin pins in place on their second transfer; the launch call "
                      "(sb200_kernel_launch_from_host) uploads A, B, C, bias by row blocks with the GEMM of each block behind "
                      "its rows; then the download of D",
               "direct_operator_pinned": {"value": flops_step / (ms3 / s3 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms3 / s3,
                                          "api": "sb200_gemm_f32_host on pinned buffers: copies, row-block GEMMs and copy-out overlapped"},
               "direct_operator_pageable": {"value": flops_step / (ms5 / 3 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms5 / 3,
                                            "api": "sb200_gemm_f32_host on pageable buffers (staged copier)"}}
        for v in vecs:
            v.free()
        del hA, hB, hC, hD, pA, pB, pC, pD
    else:
        from spoc_b200.sharding import DeviceGroup
        torch.cuda.synchronize()
        dist.barrier(group=host_group)
        if rank == 0:
          try:
              Mg = M * world
              gA, gC, gD = (np.empty(Mg * K, np.float32), np.empty(Mg * N, np.float32), np.empty(Mg * N, np.float32))
              gB, gbias = B.cpu().numpy(), bias.cpu().numpy()
              blockA, blockC = A.cpu().numpy(), Cm.cpu().numpy()
              for r in range(world):                  # any finite data: the rate does not depend on the values
                  gA[r * M * K:(r + 1) * M * K] = blockA
                  gC[r * M * N:(r + 1) * M * N] = blockC
              grp = DeviceGroup(list(range(world)))
              call = lambda: grp.gemm_host(L.MODE_3XTF32, Mg, N, K, gA, gB, gD, alpha=1.5, c=gC, beta=0.5, bias=gbias, act=L.ACT_RELU)
              call()
              call()    # the group pins a host array in place when it is handed over a second time: in the warm-up
              sg = 3
              t0 = time.perf_counter()
              for _ in range(sg):
                  call()
              ms_g = (time.perf_counter() - t0) / sg * 1e3
              # the same call on pinned host memory: plain DMA, no staging copies on the host cores
              pinned = {}
              try:
                  tp = [torch.from_numpy(x).pin_memory() for x in (gA, gB, gC, gD)]
                  nA, nB, nC, nD = (t.numpy() for t in tp)
                  callp = lambda: grp.gemm_host(L.MODE_3XTF32, Mg, N, K, nA, nB, nD, alpha=1.5, c=nC, beta=0.5, bias=gbias,
                                                act=L.ACT_RELU)
                  callp()
                  t0 = time.perf_counter()
                  for _ in range(sg):
                      callp()
                  ms_p = (time.perf_counter() - t0) / sg * 1e3
                  pinned = {"value": world * flops_step / (ms_p * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_p,
                            "identical_to_pageable": bool(np.array_equal(nD, gD))}
                  del tp, nA, nB, nC, nD
              except Exception as ex:
                  pinned = {"error": f"{type(ex).__name__}: {ex}"}
              # the block of rank 0 must equal what this rank's own operator produced for the same rows
              gemm(L.MODE_3XTF32)
              torch.cuda.synchronize()
              same = bool(np.array_equal(gD[:M * N], D.cpu().numpy()))
              grp.close()
              e2e = {"value": world * flops_step / (ms_g * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_g,
                     "h2d_bytes_per_step": 4 * (Mg * K + K * N + Mg * N + N), "d2h_bytes_per_step": 4 * Mg * N,
                     "api": "sb200_gemm_sharded_host on a group of all GPUs, one process (rank 0), host operands of "
                            f"{Mg} rows in ordinary memory, which the group pins in place on their second use: B over PCIe once "
                            "then NCCL broadcast, each GPU moves its own rows; wall clock of the call",
                     "first_block_identical_to_single_gpu": same, "pinned_host_operands": pinned,
                     "host_io_note": "perfect weak scaling of this step needs world x 67 GB/s of host memory traffic to and from "
                                     "the GPUs (1.07 GB per GPU per 16 ms); one process's pageable buffers are staged through "
                                     "pinned slots by host threads, which multiplies the host-side memory traffic by about four"}
              del gA, gC, gD
          except Exception as ex:  # the line must still be printed: say what failed
            e2e = {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "error": f"{type(ex).__name__}: {ex}"}
        dist.barrier(group=host_group)

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
                                  "traffic": 4 * (536.9e6 + 228.2e6),
                                  "traffic_unit": "bytes per launch (ncu capture at 2^26 elements, scaled x4)",
                                  "peak_source": f"{peaks['source']} copy bandwidth",
                                  "frac_of_nominal_8TBs": gbs / 8000.0}}
        # the same chain end to end through the plugin path: host vectors (pinned in place by the plugin from their
        # second transfer), the launch call uploads, computes and sends d back chunk by chunk
        try:
            from spoc_b200 import Vector, run_vectors, dims1d, sarek_ir
            import numpy as np
            hv = [Vector(backend, np.zeros(MAP_N, dtype=np.float32)) for _ in range(3)]     # d, b, c
            hv[1].host[:] = 0.25
            hv[2].host[:] = 0.5
            chain_ir = sarek_ir.chain_fused_ir(3.0)

            def map_step():
                hv[1].location = hv[2].location = Vector.CPU
                run_vectors(backend, device=dev, ir=chain_ir, args=hv, block=dims1d(256), grid=dims1d(MAP_N // 256))
                hv[0].to_array()

            ms_m, _, _ = timed(map_step, 3, 3)
            ok_m = bool(np.all(hv[0].host[:: 1 << 16] == np.float32((0.25 + 3.0 * 0.5) ** 2 + 0.25)))
            fused_map["e2e"] = {"ms_per_step": ms_m / 3, "value": 12.0 * MAP_N / (ms_m / 3 * 1e-3) / 1e9, "unit": "GB/s",
                                "h2d_bytes_per_step": 8 * MAP_N, "d2h_bytes_per_step": 4 * MAP_N, "result_ok": ok_m,
                                "api": "Execute.run_vectors mirror on the fused chain's IR with host vectors b, c, d of 1 GiB each: "
                                       "sb200_kernel_launch_from_host moves b and c up, runs the kernel and sends d back in 16 "
                                       "chunks; bound by PCIe (2 GiB up beside 1 GiB down)"}
            for v in hv:
                v.free()
            del hv
        except Exception as ex:  # the line must still be printed
            fused_map["e2e"] = {"error": f"{type(ex).__name__}: {ex}"}

    # ---- the other kernels of the path, the TF32 yardstick, the small configuration (one GPU only) -------------
    reductions = small_triad = cfg1 = tf32_yardstick = None
    if world == 1:
        from spoc_b200 import sarek_ir, dims1d, dims2d
        from spoc_b200.plugin import RSA_Buffer, RSA_Int32, RSA_Float32, _Memory
        lang = backend.supported_source_langs[0]
        buf_of = lambda t: _Memory.Buffer(dev.id, t.data_ptr(), t.numel(), 4)
        # block tree reductions over the same 2^28-element vectors (benchmarks/bench_reduction.ml, bench_dot_product.ml)
        nblocks = MAP_N // 256
        part = torch.empty(nblocks, dtype=torch.float32, device=tdev)
        reductions = {}
        for kind, vecs_in, bytes_elem in (("dot", (b, c), 8.0), ("sum", (b,), 4.0)):
            rs_args = []
            for t in vecs_in + (part,):
                rs_args += [RSA_Buffer(buf_of(t), t.numel()), RSA_Int32(t.numel())]
            rs_args.append(RSA_Int32(MAP_N))
            src = sarek_ir.block_reduce_ir(kind, 256)
            fn = lambda: backend.run_source(source=src, lang=lang, kernel_name="k", block=dims1d(256), grid=dims1d(nblocks),
                                            shared_mem=1024, args=rs_args)
            msr, lr, _ = timed(fn, 10, 3)
            g = (bytes_elem * MAP_N + 4.0 * nblocks) / (msr / 10 * 1e-3) / 1e9
            reductions["dot_product" if kind == "dot" else "reduce_sum"] = {
                "value": g, "unit": "GB/s", "ms_per_step": msr / 10, "launches_per_step": lr / 10,
                "frac_of_measured_hbm": g / peaks["hbm_gbs"], "frac_of_nominal_8TBs": g / NOMINAL_HBM_GBS}
        # stream_triad at the reference's own small benchmark size (10^6 elements): launch-latency territory; one launch
        n_small = 1_000_000
        tri_args = []
        for t in (d, b, c):
            tri_args += [RSA_Buffer(buf_of(t), n_small), RSA_Int32(n_small)]
        tri_args += [RSA_Float32(3.0), RSA_Int32(n_small)]
        tri_src = sarek_ir.stream_triad_ir()
        tri = lambda: backend.run_source(source=tri_src, lang=lang, kernel_name="sarek_kern", block=dims1d(256),
                                         grid=dims1d((n_small + 255) // 256), shared_mem=0, args=tri_args)
        mst, lt, _ = timed(tri, 200, 20)
        # the reference's own protocol: 5 warm-ups, then 20 x (launch + device synchronise) by the host clock, median
        # (benchmarks/benchmark_runner.ml:24-30, benchmarks/common.ml:222-232)
        walls = []
        for it in range(25):
            t0 = time.perf_counter()
            tri()
            _check(lib.sb200_device_synchronize(dev.id))
            if it >= 5:
                walls.append((time.perf_counter() - t0) * 1e6)
        small_triad = {"n": n_small, "us_per_launch": mst / 200 * 1e3, "launches_per_step": lt / 200,
                       "launch_plus_sync_median_us": statistics.median(walls),
                       "reference_published_median_us": {"value": 14.07, "where": "benchmarks/results/drangleic_stream_triad_1000000_2026-01-12T17-51-33.json, CUDA backend on an RTX 5070 Ti (other hardware)"},
                       "value": 12.0 * n_small / (mst / 200 * 1e-3) / 1e9, "unit": "GB/s",
                       "note": "through run_source on the kernel's IR, back to back on one stream (inputs stay in L2 at this size)"}
        del b, c, d, part
        # configuration 1: 1024^3 through the tiled kernel's IR (cache-resident: a parity and CPU-baseline anchor)
        S1 = 1024
        t1 = [torch.empty(S1 * S1, dtype=torch.float32, device=tdev) for _ in range(3)]
        fill(t1[0], 1, 0)
        fill(t1[1], 2, 0)
        mm_args = []
        for t in t1:
            mm_args += [RSA_Buffer(buf_of(t), t.numel()), RSA_Int32(t.numel())]
        mm_args += [RSA_Int32(S1)] * 3
        mm_src = sarek_ir.matmul_tiled_ir()
        cfg1 = {"workload": "gemm M=N=K=1024 (BASELINE configs[0]) through the matrix_mul_tiled IR, block 16x16, grid 64x64"}
        for mode, label in ((L.MODE_3XTF32, "3xtf32"), (L.MODE_TF32, "tf32")):
            backend.set_mode(mode)
            mm = lambda: backend.run_source(source=mm_src, lang=lang, kernel_name="sarek_kern", block=dims2d(16, 16),
                                            grid=dims2d(S1 // 16, S1 // 16), shared_mem=0, args=mm_args)
            ms1, _, _ = timed(mm, 100, 10)
            cfg1[label] = {"us_per_launch": ms1 / 100 * 1e3, "value": 2.0 * S1 ** 3 / (ms1 / 100 * 1e-3) / 1e12, "unit": "TFLOP/s"}
        backend.set_mode(L.MODE_3XTF32)
        del t1
        # yardstick: a TF32 library GEMM (cuBLAS through torch.matmul with TF32 allowed) at 8192^3, best of 10 and 4 s
        # back to back — the measured dense-TF32 rate of this GPU, beside the nominal figure.  A yardstick only.
        ya = torch.empty(M, K, dtype=torch.float32, device=tdev).uniform_(-1, 1)
        yb = torch.empty(K, N, dtype=torch.float32, device=tdev).uniform_(-1, 1)
        yc = torch.empty(M, N, dtype=torch.float32, device=tdev)
        prev_tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        time.sleep(0.5)
        best = 1e9
        for _ in range(3):
            torch.matmul(ya, yb, out=yc)
        torch.cuda.synchronize()
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(ya, yb, out=yc)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        t_y = time.time()
        cnt = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        while time.time() - t_y < 4.0:
            for _ in range(20):
                torch.matmul(ya, yb, out=yc)
            cnt += 20
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / cnt
        torch.backends.cuda.matmul.allow_tf32 = prev_tf32
        tf32_yardstick = {"library": "cuBLAS via torch.matmul, allow_tf32", "burst_tflops": flops_step / (best * 1e-3) / 1e12,
                          "sustained_tflops": flops_step / (sustained_ms * 1e-3) / 1e12, "nominal_tflops": NOMINAL_TF32_TFLOPS}
        del ya, yb, yc
        torch.cuda.empty_cache()
        for rf in (roofline, tf32_mode["roofline"]):
            rf["frac_of_nominal_tf32_peak"] = rf["achieved"] / NOMINAL_TF32_TFLOPS
            rf["frac_of_measured_tf32_library_sustained"] = rf["achieved"] / tf32_yardstick["sustained_tflops"]
            rf["frac_of_measured_tf32_library_burst"] = rf["achieved"] / tf32_yardstick["burst_tflops"]

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        workers = max(1, (os.cpu_count() or 2) - 1)
        step, ids = cpu_slab_rate(workers, target_s=12.0)
        dt = step()
        cpu_baseline = {"value": 2.0 * K * ids / dt / 1e12, "unit": "TFLOP/s", "cores": workers, "kind": "port",
                        "sample": f"first {ids} output elements ({ids / N:.2f} rows) of the same 8192^3 problem, "
                                  f"{dt:.1f} s, extrapolated; C restatement of Sarek Native's naive kernel with the epilogue"}
        # the two configurations a CPU can run in full: 1024^3 on Native's tiled (barrier) path with all cores
        # (sarek/sarek/Sarek_cpu_runtime.ml:1025), and the 2^28-element chain as two unfused kernels
        import numpy as np
        O = oracle_lib()
        olib = O.load()
        a1, b1, c1 = O.fill(1024 * 1024, SEED, 1), O.fill(1024 * 1024, SEED, 2), np.zeros(1024 * 1024, np.float32)
        t0 = time.perf_counter()
        olib.so_par_matmul_tiled(a1, b1, c1, 1024, 1024, 1024, 0, 64 * 64, workers + 1)
        dt1 = time.perf_counter() - t0
        cpu_baseline["config_1024cubed_tiled"] = {"value": 2.0 * 1024 ** 3 / dt1 / 1e12, "unit": "TFLOP/s", "seconds": dt1,
                                                  "cores": workers + 1, "sample": "the full problem, tiled kernel, barrier path"}
        hb, hc = O.fill(MAP_N, SEED, 2), O.fill(MAP_N, SEED, 3)
        ha, hd = np.empty(MAP_N, np.float32), np.empty(MAP_N, np.float32)
        t0 = time.perf_counter()
        olib.so_par_chain_triad_square(hd, ha, hb, hc, 3.0, MAP_N, workers)
        dt2 = time.perf_counter() - t0
        cpu_baseline["config_chain_2p28_unfused"] = {"value": 12.0 * MAP_N / dt2 / 1e9, "unit": "GB/s (12 B per element, as the fused GPU pass)",
                                                     "seconds": dt2, "cores": workers,
                                                     "sample": "the full 2^28 elements, two unfused kernels (the second reads the stored intermediate)"}
        del hb, hc, ha, hd

    # ---- the strong-scaling configurations, at every N -----------------------------------------------------------
    try:
        del A, Cm
    except NameError:
        pass
    del B, D
    torch.cuda.empty_cache()
    skinny = skinny_leg(ctx, max(3, min(args.steps, 10)), 3)
    gather = gather_leg(ctx, args.gather_size, 3, 1)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3 (f32 in/out)",
            "data": "synthetic",
            "config": make_config(args),
            "arm": {"mode": "3xTF32 split accumulation on tcgen05 tensor cores", "preload_s": args.preload_s},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "burst": burst, "tf32_mode": tf32_mode, "f16_split_mode": f16_split_mode, "f16_single_mode": f16_single_mode, "mixed_mode": mixed_mode, "fused_map": fused_map, "b_broadcast_ms": bcast_ms,
            "reductions": reductions, "stream_triad_1e6": small_triad, "config_1024cubed": cfg1, "tf32_yardstick": tf32_yardstick,
            "skinny_65536x4096x4096": skinny, f"gather_{args.gather_size}cubed": gather,
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
    if args.case in ("gemm3", "gemm1", "gemm4", "gemm5"):
        mode = {"gemm3": L.MODE_3XTF32, "gemm1": L.MODE_TF32, "gemm4": L.MODE_3XF16, "gemm5": L.MODE_3XMIXED}[args.case]
        Mr = args.rows or S        # --rows: a row block of the square problem (what one GPU of a group computes)
        bufs = [torch.empty(n, dtype=torch.float32, device=tdev) for n in (Mr * S, S * S, Mr * S, Mr * S)]
        bias = torch.empty(S, dtype=torch.float32, device=tdev)
        for i, t in enumerate(bufs[:3]):
            _check(lib.sb200_fill_f32(dev.id, stream, t.data_ptr(), t.numel(), SEED, i + 1, 0, 1.0, 0))
        _check(lib.sb200_fill_f32(dev.id, stream, bias.data_ptr(), S, SEED, 4, 1, 1.0, 0))
        fn = lambda: _check(lib.sb200_gemm_f32(dev.id, stream, mode, Mr, S, S, bufs[0].data_ptr(), S, bufs[1].data_ptr(), S,
                                               bufs[3].data_ptr(), S, 1.5, bufs[2].data_ptr(), S, 0.5, bias.data_ptr(), 1))
        work, unit = 2.0 * Mr * S * S / 1e12, "TFLOP/s"
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
    print(json.dumps({"case": args.case, "size": S, "rows": getattr(args, "rows", 0) or S, "ms_per_call": ms, "rate": work / (ms * 1e-3), "unit": unit}), flush=True)


class Ctx:
    """What the multi-GPU legs share: the library, this rank's device and stream, the process group."""

    def __init__(self, rank: int, local_rank: int, world: int):
        import torch
        import torch.distributed as dist
        from spoc_b200 import Backend, _lib as L
        self.torch, self.dist, self.L = torch, dist, L
        self.lib = L.load()
        self.rank, self.local_rank, self.world = rank, local_rank, world
        torch.cuda.set_device(local_rank)
        if world > 1 and not dist.is_initialized():
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        self.backend = Backend()
        self.backend.Device.init()
        self.dev = self.backend.Device.get(local_rank)
        self.backend.Device.set_current(self.dev)
        self.tdev = torch.device("cuda", local_rank)
        self.stream = torch.cuda.current_stream().cuda_stream

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.tdev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, flag: bool) -> bool:
        if self.world == 1:
            return flag
        t = self.torch.tensor([1 if flag else 0], device=self.tdev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def timed(self, fn, steps: int, warmup: int) -> float:
        """ms per step: CUDA events on the launch stream, a barrier and a synchronise on both sides, max over ranks."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1) / steps)


def oracle_parity(ctx, D_rows_fn, A, B, M_rows, N, K, row_ids, a_row_fn, c_row_fn, bias, alpha, beta, act, bound_scale, mode_is_3x=True):
    """Checker, outside every timed region: sampled rows x 64 random columns of a device result against the CPU
    oracle (tests/oracle_lib.py).  The oracle sees B's sampled columns as the device holds them and regenerates the
    rows of A and C with the host generator.  Returns (ok, worst error / bound)."""
    import math
    import numpy as np
    O = oracle_lib()
    torch = ctx.torch
    rng = np.random.default_rng(1234 + ctx.rank)
    cols = np.sort(rng.choice(N, size=min(64, N), replace=False))
    tcols = torch.from_numpy(cols).to(ctx.tdev)
    b_c = B.view(K, N).index_select(1, tcols).contiguous().cpu().numpy()            # K x 64, as the device holds B
    a_s = np.vstack([a_row_fn(r) for r in row_ids])                                  # rows x K
    c_s = np.vstack([c_row_fn(r)[cols] for r in row_ids]) if c_row_fn else None
    bias_c = np.ascontiguousarray(bias[cols]) if bias is not None else None
    ref = O.gemm(np.ascontiguousarray(a_s).ravel(), np.ascontiguousarray(b_c).ravel(), len(row_ids), len(cols), K, alpha, beta,
                 None if c_s is None else np.ascontiguousarray(c_s).ravel(), bias_c, act)
    got = np.vstack([D_rows_fn(r)[cols] for r in row_ids])
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) or 1.0
    err = float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(np.abs(ref), rms)))
    bound = (1e-5 * math.sqrt(K) if mode_is_3x else 2e-3) * bound_scale
    return err <= bound, err / bound


def gather_leg(ctx, S: int, steps: int, warmup: int) -> dict:
    """Strong scaling of the large square GEMM with epilogue and a gathered result (BASELINE configs[4]): M = N = K = S,
    rows of A/C/D split over the ranks, B replicated by NCCL broadcast.  Two ways to leave the whole D on every GPU
    are timed: the GEMM followed by an NCCL all-gather of the row blocks, and the GEMM whose epilogue stores each
    tile into every GPU's copy (peer stores over NVLink).  The two forms alternate over three rounds so that a
    drift of the clocks under the power cap hits both alike; each form's figure is the median of its rounds.  Sampled rows
    of every rank's gathered copy — rows computed by every rank — are checked against the CPU oracle."""
    import numpy as np
    torch, dist, L, lib = ctx.torch, ctx.dist, ctx.L, ctx.lib
    from spoc_b200.plugin import _check
    from spoc_b200.sharding import row_block, partition
    dev, stream, rank, world, tdev = ctx.dev, ctx.stream, ctx.rank, ctx.world, ctx.tdev
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
    D_nccl = torch.empty(S * S, dtype=torch.float32, device=tdev)        # gathered by NCCL
    D_own = ctx.backend.Memory.alloc(dev, S * S, np.float32)              # gathered by the epilogue (IPC-shareable memory)
    copies, opened = [D_own.ptr], []
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

    rounds = {"nccl": [], "fused": []}
    for rnd in range(3):
        rounds["nccl"].append(ctx.timed(step_nccl, steps, warmup if rnd == 0 else 1))
        rounds["fused"].append(ctx.timed(step_fused, steps, warmup if rnd == 0 else 1))
    ms_nccl, ms_fused = statistics.median(rounds["nccl"]), statistics.median(rounds["fused"])
    # the two gathered results must agree bit for bit on this rank (compared in slabs: no third 4 GiB buffer)
    same = True
    slab = max(1, (1 << 28) // S) * S
    own_view = torch.empty(min(slab, S * S), dtype=torch.float32, device=tdev)
    for off in range(0, S * S, slab):
        cnt = min(slab, S * S - off)
        _check(lib.sb200_memcpy_dtod(dev.id, own_view.data_ptr(), D_own.ptr + 4 * off, 4 * cnt))
        same = same and bool(torch.equal(own_view[:cnt], D_nccl[off:off + cnt]))
    same = ctx.all_true(same)
    # oracle check of this rank's gathered copy: four rows out of every rank's block
    O = oracle_lib()
    rng = np.random.default_rng(99)
    row_ids = []
    for f, cnt in partition(S, world):
        if cnt:
            row_ids += sorted(set([f, f + cnt - 1] + (f + rng.integers(0, cnt, 2)).tolist()))
    hbias = bias.cpu().numpy()

    def d_row(r):
        out = np.empty(S, np.float32)
        _check(lib.sb200_memcpy_dtoh(dev.id, out.ctypes.data_as(C.c_void_p), D_own.ptr + 4 * r * S, 4 * S))
        return out

    ok, rel = oracle_parity(ctx, d_row, A, B, S, S, S, row_ids, lambda r: O.fill(S, SEED, 1, first=r * S),
                            lambda r: O.fill(S, SEED, 3, first=r * S), hbias, 1.5, 0.5, 1, 1.5 * 2 ** 0.5)
    ok = ctx.all_true(ok)
    rel = ctx.max_over_ranks(rel)
    # the fused form once more in the mixed mode (main term TF32, cross terms fp16), checked against the oracle likewise
    def step_fused_mixed():
        _check(lib.sb200_gemm_f32_gather(dev.id, stream, L.MODE_3XMIXED, rows, S, S, A.data_ptr(), S, B.data_ptr(), S, ptrs,
                                         len(copies), r0, S, 1.5, Cm.data_ptr(), S, 0.5, bias.data_ptr(), L.ACT_RELU))

    ms_mixed = ctx.timed(step_fused_mixed, steps, 1)
    ok_m, rel_m = oracle_parity(ctx, d_row, A, B, S, S, S, row_ids, lambda r: O.fill(S, SEED, 1, first=r * S),
                                lambda r: O.fill(S, SEED, 3, first=r * S), hbias, 1.5, 0.5, 1, 1.5 * 2 ** 0.5)
    ok_m = ctx.all_true(ok_m)
    rel_m = ctx.max_over_ranks(rel_m)
    ctx.barrier()
    for pp in opened:
        _check(lib.sb200_ipc_close(dev.id, pp))
    ctx.backend.Memory.free(D_own)
    del A, Cm, B, D_nccl, own_view
    torch.cuda.empty_cache()
    flops = 2.0 * S ** 3
    nvlink_bytes = 4.0 * rows * S * (world - 1)       # what this rank's epilogue stores into its peers' copies per step
    return {
        "metric": f"fp32_gemm_fused_epilogue_{S}cubed_gathered", "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "scaling": "strong", "dtype": "tf32x3 (f32 in/out)",
        "workload": f"gemm M=N=K={S} with epilogue (BASELINE configs[4]), rows of A/C/D split over the GPUs, whole D on every GPU",
        "value": flops / (ms_fused * 1e-3) / 1e12, "ms_per_step": ms_fused,
        "gemm_then_nccl_all_gather": {"value": flops / (ms_nccl * 1e-3) / 1e12, "ms_per_step": ms_nccl, "rounds_ms": rounds["nccl"]},
        "gather_fused_in_epilogue": {"value": flops / (ms_fused * 1e-3) / 1e12, "ms_per_step": ms_fused, "rounds_ms": rounds["fused"],
                                     "peer_store_bytes_per_gpu": nvlink_bytes,
                                     "peer_store_gbs_per_gpu": nvlink_bytes / (ms_fused * 1e-3) / 1e9},
        "gather_fused_in_epilogue_mixed_mode": {"value": flops / (ms_mixed * 1e-3) / 1e12, "ms_per_step": ms_mixed,
                                                "parity_ok": ok_m, "parity_worst_over_bound": rel_m,
                                                "note": "SB200_MODE_3XMIXED, one timed pass after one warm-up step; the mode's "
                                                        "magnitude scan and panel passes are inside the step"},
        "results_identical": same, "parity_ok": ok, "parity_worst_over_bound": rel,
        "parity": f"{len(row_ids)} rows (every rank's block) x 64 columns of each rank's gathered copy against the CPU oracle, "
                  "bound 1e-5*sqrt(K)*1.5*sqrt(2) relative to max(|ref|, rms)"}


def run_gather(args, rank: int, local_rank: int, world: int) -> None:
    ctx = Ctx(rank, local_rank, world)
    out = gather_leg(ctx, args.size, args.steps, max(args.warmup, 1))
    if rank == 0:
        out.update({"warmup": max(args.warmup, 1), "higher_is_better": True, "data": "synthetic",
                    "config": {"workload": out["workload"]}})
        print(json.dumps(out), flush=True)
    if world > 1:
        ctx.dist.destroy_process_group()


def skinny_leg(ctx, steps: int, warmup: int) -> dict:
    """Strong scaling of the skinny GEMM (BASELINE configs[3]): C = A.B with M = 65536, N = K = 4096, rows of A drawn
    from N(0,1), B from N(0,1/sqrt(K)); rows of A and C split over the ranks, B broadcast from rank 0 (NCCL).  Timed
    with B already on every GPU and with the broadcast of B inside every timed step, in both modes, the two variants
    alternating over three rounds (median); sampled rows of every rank's block are checked against the CPU oracle."""
    import math
    import numpy as np
    torch, dist, L, lib = ctx.torch, ctx.dist, ctx.L, ctx.lib
    from spoc_b200.plugin import _check
    from spoc_b200.sharding import row_block
    dev, stream, rank, world, tdev = ctx.dev, ctx.stream, ctx.rank, ctx.world, ctx.tdev
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
    O = oracle_lib()
    out, parity_ok, parity_rel = {}, True, 0.0
    for mode, label in ((L.MODE_3XTF32, "3xtf32"), (L.MODE_TF32, "tf32"), (L.MODE_3XMIXED, "mixed")):
        def gemm():
            _check(lib.sb200_gemm_f32(dev.id, stream, mode, rows, Nn, Kk, A.data_ptr(), Kk, B.data_ptr(), Nn, Cm.data_ptr(), Nn,
                                      1.0, 0, 0, 0.0, 0, L.ACT_NONE))

        def gemm_after_broadcast():
            if world > 1:
                dist.broadcast(B, src=0)
            gemm()

        # the two variants alternate over three rounds after a short pre-load, so that the settling of the clocks
        # under the power cap hits both alike; the figure of each is the median of its rounds
        t_pre = time.time()
        while time.time() - t_pre < 0.3:
            for _ in range(10):
                gemm()
            torch.cuda.synchronize()
        rounds = {"b_resident": [], "b_broadcast_timed": []}
        for rnd in range(3):
            for name, fn in (("b_resident", gemm), ("b_broadcast_timed", gemm_after_broadcast)):
                rounds[name].append(ctx.timed(fn, steps, max(warmup, 3) if rnd == 0 else 1))
        for name, ms_list in rounds.items():
            ms = statistics.median(ms_list)
            out.setdefault(label, {})[name] = {"ms_per_step": ms, "value": 2.0 * Mt * Nn * Kk / (ms * 1e-3) / 1e12,
                                              "rounds_ms": ms_list}
        rng = np.random.default_rng(7 + rank)
        row_ids = sorted(set([0, rows - 1] + rng.integers(0, rows, 6).tolist()))
        hC = Cm.view(rows, Nn)
        ok, rel = oracle_parity(ctx, lambda r: hC[r].cpu().numpy(), A, B, rows, Nn, Kk, row_ids,
                                lambda r: O.fill(Kk, SEED, 1, kind=2, first=(r0 + r) * Kk), None, None, 1.0, 0.0, 0, 1.0,
                                mode_is_3x=(mode in (L.MODE_3XTF32, L.MODE_3XMIXED)))
        parity_ok = parity_ok and ok
        parity_rel = max(parity_rel, rel)
    parity_ok = ctx.all_true(parity_ok)
    parity_rel = ctx.max_over_ranks(parity_rel)
    del A, Cm, B
    torch.cuda.empty_cache()
    return {"metric": "fp32_gemm_65536x4096x4096_row_sharded", "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "scaling": "strong", "dtype": "tf32x3, tf32 and tf32 + 2 x f16 cross terms (f32 in/out)",
            "workload": "gemm M=65536 N=K=4096 (BASELINE configs[3]), A ~ N(0,1), B ~ N(0,1/sqrt(K)), rows of A/C split over the "
                        "GPUs, B broadcast from rank 0 (64 MiB, NCCL)",
            "value": out["3xtf32"]["b_resident"]["value"], "ms_per_step": out["3xtf32"]["b_resident"]["ms_per_step"],
            "modes": out, "parity_ok": parity_ok, "parity_worst_over_bound": parity_rel,
            "parity": "8 rows of every rank's block x 64 columns against the CPU oracle in the three modes "
                      "(bounds 1e-5*sqrt(K) for 3xTF32 and the mixed mode, 2e-3 for TF32, relative to max(|ref|, rms))"}


def run_skinny(args, rank: int, local_rank: int, world: int) -> None:
    ctx = Ctx(rank, local_rank, world)
    out = skinny_leg(ctx, args.steps, args.warmup)
    if rank == 0:
        out.update({"warmup": max(args.warmup, 3), "higher_is_better": True, "data": "synthetic",
                    "config": {"workload": out["workload"]}})
        print(json.dumps(out), flush=True)
    if world > 1:
        ctx.dist.destroy_process_group()


def _keep_stdout_for_the_result_line() -> None:
    """Libraries that write to file descriptor 1 themselves (NCCL prints its version there) must not add lines to the
    one-line result: descriptor 1 is pointed at stderr for them, and Python's stdout keeps the real one."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(saved, "w", buffering=1)


def main() -> None:
    _keep_stdout_for_the_result_line()
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm8192", choices=["gemm8192", "gather", "skinny"],
                    help="gemm8192: the headline run; gather: large square GEMM with the result gathered on every GPU; "
                         "skinny: 65536x4096x4096 GEMM, rows split over the ranks, B broadcast")
    ap.add_argument("--case", default=None, choices=["gemm3", "gemm1", "gemm4", "gemm5", "map", "transfer", "tiles"],
                    help="profiler-sized single-operator run (square size --size; map uses size^2 elements)")
    ap.add_argument("--size", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=0, help="--case gemm*: M (default: --size); N = K = --size")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather-size", type=int, default=32768, help="M = N = K of the gathered-result configuration in the default run")
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
