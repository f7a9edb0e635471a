"""The benchmark harness mirror writes the reference's result schema (benchmarks/output.ml:39-89): checked here against
the keys of a result file the reference itself published, whose structure is restated below."""
import numpy as np
import pytest

from spoc_b200 import sarek_bench as SB

# keys of benchmarks/results/drangleic_stream_triad_1000000_2026-01-12T17-51-33.json in the reference
TOP = {"benchmark", "system", "results"}
BENCHMARK = {"name", "timestamp", "git_commit", "parameters"}
PARAMETERS = {"size", "block_size", "iterations", "warmup"}
SYSTEM = {"hostname", "os", "kernel", "cpu", "memory_gb", "devices"}
RESULT = {"verified", "throughput_gflops", "device_id", "device_name", "framework", "iterations", "mean_ms", "stddev_ms",
          "median_ms", "min_ms", "max_ms"}


def test_result_document_has_the_reference_schema():
    r = SB.device_result(0, "NVIDIA B200", "B200", [0.02, 0.01, 0.03], 12.0e6, "median", True)
    doc = SB.to_json("stream_triad", 1_000_000, 256, 3, 5, SB.system_info([{"id": 0, "name": "NVIDIA B200", "framework": "B200",
                                                                           "memory_gb": 178.0}]), [r], timestamp="2026-01-01T00:00:00Z")
    assert set(doc) == TOP and set(doc["benchmark"]) == BENCHMARK and set(doc["benchmark"]["parameters"]) == PARAMETERS
    assert set(doc["system"]) == SYSTEM and set(doc["system"]["cpu"]) == {"model", "cores", "threads"}
    assert set(doc["results"][0]) == RESULT
    assert r["median_ms"] == 0.02 and r["min_ms"] == 0.01 and r["max_ms"] == 0.03
    assert r["throughput_gflops"] == pytest.approx(12.0e6 / 0.02e-3 / 1e9)   # GB/s from the median, as bench_stream_triad.ml:153-156


def test_failed_and_empty_results_are_filtered_like_the_reference():
    ok = SB.device_result(0, "d", "B200", [1.0], 1.0, "median", True)
    bad = dict(ok, median_ms=0.0, verified=False)
    empty = dict(ok, iterations=[])
    doc = SB.to_json("vector_add", 10, 256, 1, 0, SB.system_info([]), [ok, bad, empty])
    assert doc["results"] == [ok]


@pytest.mark.parametrize("name,size", [("vector_add", 1000), ("stream_triad", 1000), ("matrix_mul", 24), ("matrix_mul_tiled", 24)])
def test_host_cases_follow_the_reference_patterns(name, size):
    c = SB.host_case(name, size)
    if name == "stream_triad":
        assert c["vecs"][1][101] == np.float32(0.01) and c["vecs"][2][99] == np.float32(0.0) and c["tol"] == 1e-5
        assert c["expected"][5] == pytest.approx(0.05 + 0.06 * 3.0, abs=1e-6)
    if name.startswith("matrix_mul"):
        assert c["vecs"][0][13] == np.float32(0.3) and c["vecs"][1][9] == np.float32(0.0) and c["work"] == 2.0 * size ** 3
    assert len(c["vecs"][c["out"]]) == len(c["expected"])


@pytest.mark.gpu
@pytest.mark.parametrize("name,size", [("vector_add", 100_000), ("stream_triad", 1_000_000), ("matrix_mul", 128), ("matrix_mul_tiled", 256)])
def test_benchmarks_run_and_verify_on_the_gpu(backend, device, name, size):
    r = SB.run_one(backend, device, name, size, iterations=5, warmup=2)
    assert r["verified"] is True and len(r["iterations"]) == 5 and r["throughput_gflops"] > 0
