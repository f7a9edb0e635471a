"""The reference's benchmark protocol for the kernels of this path, with results in the reference's JSON schema.

    python -m spoc_b200.sarek_bench --bench stream_triad --sizes 1000000,10000000 --output results/

Mirrors what `benchmarks/benchmark_runner.ml` and the per-kernel drivers do on a device
(benchmarks/bench_vector_add.ml, bench_stream_triad.ml, bench_matrix_mul.ml, bench_matrix_mul_tiled.ml): host data
from the driver's own index pattern, `warmup` untimed launches, `iterations` timed ones — each a launch plus a device
synchronise by the host clock (benchmarks/common.ml:217-235) —, verification against the driver's host baseline with
its tolerance, throughput from the median (the minimum for vector_add, as that driver does), and one JSON file per
(benchmark, size) in the schema of benchmarks/output.ml:39-89 and benchmarks/system_info.ml:202-240, so that the
reference's `to_web` / `aggregate` tools ingest the files unchanged.  The kernels run through `run_vectors` on the
kernel's IR: the same path a `[%kernel]` caller takes.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import platform
import socket
import statistics
import subprocess
import time

import numpy as np

from . import sarek_ir
from .plugin import Backend, Vector, dims1d, dims2d, run_vectors

BENCHES = ("vector_add", "stream_triad", "matrix_mul", "matrix_mul_tiled")


def host_case(name: str, size: int):
    """(ir, vectors as numpy arrays, scalars, block, grid, shared_mem, expected, tolerance, work per launch) for one
    benchmark at one size, with the reference driver's data pattern and host baseline."""
    if name == "vector_add":          # bench_vector_add.ml:68-71,113-125
        i = np.arange(size, dtype=np.float64)
        a, b = (i * 0.001).astype(np.float32), (i * 0.002).astype(np.float32)
        exp = a.astype(np.float64) + b.astype(np.float64)
        return dict(ir=sarek_ir.vector_add_ir(), vecs=[a, b, np.zeros(size, np.float32)], out=2, scalars=[("int32", size)],
                    block=dims1d(256), grid=dims1d((size + 255) // 256), shared=0, expected=exp, tol=1e-3, work=12.0 * size,
                    stat="min")
    if name == "stream_triad":        # bench_stream_triad.ml:44-49,122,153-156
        i = np.arange(size)
        b, c = ((i % 100) / 100.0).astype(np.float32), (((i + 1) % 100) / 100.0).astype(np.float32)
        exp = b.astype(np.float64) + c.astype(np.float64) * 3.0
        return dict(ir=sarek_ir.stream_triad_ir(), vecs=[np.zeros(size, np.float32), b, c], out=0,
                    scalars=[("float32", 3.0), ("int32", size)], block=dims1d(256), grid=dims1d((size + 255) // 256), shared=0,
                    expected=exp, tol=1e-5, work=12.0 * size, stat="median")
    if name in ("matrix_mul", "matrix_mul_tiled"):   # bench_matrix_mul_tiled.ml:41-52,106-141,194-226: size is the dimension
        n = size
        a = ((np.arange(n * n) % 10) / 10.0).astype(np.float32)
        b = (((np.arange(n * n) + 1) % 10) / 10.0).astype(np.float32)
        exp = (a.astype(np.float64).reshape(n, n) @ b.astype(np.float64).reshape(n, n)).ravel()
        tiled = name.endswith("tiled")
        return dict(ir=sarek_ir.matmul_tiled_ir() if tiled else sarek_ir.matmul_naive_ir(), vecs=[a, b, np.zeros(n * n, np.float32)],
                    out=2, scalars=[("int32", n)] * 3, block=dims2d(16, 16) if tiled else dims1d(256),
                    grid=dims2d((n + 15) // 16, (n + 15) // 16) if tiled else dims1d((n * n + 255) // 256),
                    shared=2 * 16 * 16 * 4 if tiled else 0, expected=exp, tol=1e-3, work=2.0 * n ** 3, stat="median")
    raise ValueError(f"unknown benchmark {name!r}; one of {BENCHES}")


def device_result(dev_id: int, dev_name: str, framework: str, times_ms: list[float], work: float, stat: str, verified: bool) -> dict:
    """One entry of `results` (benchmarks/output.ml:39-66).  `throughput_gflops` carries GFLOP/s for the matrix
    products and GB/s for the bandwidth kernels, as the reference's drivers put them there."""
    t = {"min": min(times_ms), "median": statistics.median(times_ms)}[stat]
    return {"verified": bool(verified), "throughput_gflops": work / (t * 1e-3) / 1e9 if t > 0 else 0.0, "device_id": dev_id,
            "device_name": dev_name, "framework": framework, "iterations": list(times_ms), "mean_ms": statistics.fmean(times_ms),
            "stddev_ms": statistics.pstdev(times_ms) if len(times_ms) > 1 else 0.0, "median_ms": statistics.median(times_ms),
            "min_ms": min(times_ms), "max_ms": max(times_ms)}


def system_info(devices: list[dict]) -> dict:
    """benchmarks/system_info.ml:202-240."""
    model = ""
    try:
        with open("/proc/cpuinfo") as f:
            model = next((ln.split(":", 1)[1].strip() for ln in f if ln.startswith("model name")), "")
    except OSError:
        pass
    mem_gb = 0.0
    try:
        with open("/proc/meminfo") as f:
            mem_gb = int(next(ln for ln in f if ln.startswith("MemTotal")).split()[1]) / 1048576.0
    except (OSError, StopIteration):
        pass
    threads = os.cpu_count() or 1
    return {"hostname": socket.gethostname(), "os": platform.system(), "kernel": platform.release(),
            "cpu": {"model": model, "cores": threads, "threads": threads}, "memory_gb": mem_gb, "devices": devices}


def to_json(name: str, size: int, block_size: int, iterations: int, warmup: int, system: dict, results: list[dict],
            timestamp: str | None = None, git_commit: str | None = None) -> dict:
    """benchmarks/output.ml:68-89; results with no timing or with a failed verification and zero time are dropped as
    `filter_valid_results` does (:93-99)."""
    ts = timestamp or datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
    valid = [r for r in results if r["iterations"] and not (r["median_ms"] == 0.0 and r.get("verified") is False)]
    return {"benchmark": {"name": name, "timestamp": ts, "git_commit": git_commit,
                          "parameters": {"size": size, "block_size": block_size, "iterations": iterations, "warmup": warmup}},
            "system": system, "results": valid}


def run_one(backend: Backend, device, name: str, size: int, iterations: int = 20, warmup: int = 5, framework: str = "B200") -> dict:
    case = host_case(name, size)
    vecs = [Vector(backend, v) for v in case["vecs"]]
    args = vecs + case["scalars"]
    launch = lambda: run_vectors(backend, device=device, ir=case["ir"], args=args, block=case["block"], grid=case["grid"],
                                 shared_mem=case["shared"])
    try:
        for _ in range(warmup):
            launch()
        backend.Device.synchronize(device)
        times = []
        for _ in range(iterations):
            t0 = time.perf_counter()
            launch()
            backend.Device.synchronize(device)
            times.append((time.perf_counter() - t0) * 1e3)
        got = vecs[case["out"]].to_array().astype(np.float64)
        verified = bool(np.all(np.abs(got - case["expected"]) <= case["tol"] * np.maximum(1.0, np.abs(case["expected"]))))
    finally:
        for v in vecs:
            v.free()
    return device_result(backend.Device.id(device), backend.Device.name(device), framework, times, case["work"], case["stat"], verified)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--bench", default="stream_triad", choices=BENCHES)
    ap.add_argument("--sizes", default="1000000")
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--output", default="results")
    args = ap.parse_args()
    backend = Backend()
    backend.Device.init()
    device = backend.Device.get(0)
    backend.Device.set_current(device)
    caps = backend.Device.capabilities(device)
    sysinfo = system_info([{"compute_capability": "%d.%d" % tuple(caps.get("compute_capability", (10, 0))), "id": 0,
                            "name": backend.Device.name(device), "framework": "B200",
                            "memory_gb": caps.get("total_global_mem", 0) / 2 ** 30}])
    commit = None
    try:
        commit = subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, check=True).stdout.strip() or None
    except (OSError, subprocess.CalledProcessError):
        pass
    os.makedirs(args.output, exist_ok=True)
    for size in (int(x) for x in args.sizes.split(",")):
        res = run_one(backend, device, args.bench, size, args.iterations, args.warmup)
        doc = to_json(args.bench, size, 256, args.iterations, args.warmup, sysinfo, [res], git_commit=commit)
        stamp = doc["benchmark"]["timestamp"].replace(":", "-").rstrip("Z")
        path = os.path.join(args.output, f"{sysinfo['hostname']}_{args.bench}_{size}_{stamp}.json")
        with open(path, "w") as f:
            json.dump(doc, f, indent=2)
        print(f"{args.bench} size {size}: median {res['median_ms']:.4f} ms, throughput {res['throughput_gflops']:.1f}, "
              f"verified {res['verified']} -> {path}")


if __name__ == "__main__":
    main()
