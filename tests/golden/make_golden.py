"""Generates tests/golden/reference_fixtures.json.

The reference is OCaml and cannot be run where this repository is built, so the
golden vectors are the closed-form fixtures its own tests and benchmarks use for
this path, evaluated here with numpy float64 — the arithmetic those OCaml
baselines use — independently of the C oracle:

* matmul: A[i]=(i mod 10)/10, B[i]=((i+1) mod 10)/10, expected = double triple loop
  (benchmarks/bench_matrix_mul_tiled.ml:41-52,109-112; sarek/tests/e2e/test_matrix_mul.ml:44-54), tol 1e-3
* stream_triad: B=(i mod 100)/100, C=((i+1) mod 100)/100, scalar 3.0 (benchmarks/bench_stream_triad.ml:44-49,122), tol 1e-5
* vector_add: a=i, b=2i, expected 3i (sarek/tests/e2e/test_vector_add.ml:31-49) and a=i*0.001, b=i*0.002
  (benchmarks/bench_vector_add.ml:68-71), tol 1e-3

Run: python tests/golden/make_golden.py
"""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    out = {"matmul": [], "triad": {}, "vector_add": []}
    for m, n, k in ((8, 8, 8), (32, 32, 32), (17, 23, 29), (64, 48, 40)):
        a = (np.arange(m * k) % 10) / 10.0
        b = ((np.arange(k * n) + 1) % 10) / 10.0
        exp = np.zeros((m, n))
        for row in range(m):
            for col in range(n):
                s = 0.0
                for i in range(k):
                    s = s + a[row * k + i] * b[i * n + col]
                exp[row, col] = s
        out["matmul"].append({"m": m, "n": n, "k": k, "tolerance": 1e-3, "expected": exp.ravel().tolist()})
    n = 1000
    i = np.arange(n)
    b, c = (i % 100) / 100.0, ((i + 1) % 100) / 100.0
    out["triad"] = {"n": n, "scalar": 3.0, "tolerance": 1e-5, "expected": (b + c * 3.0).tolist()}
    for scale_a, scale_b in ((1.0, 2.0), (0.001, 0.002)):
        i = np.arange(512, dtype=np.float64)
        out["vector_add"].append({"n": 512, "scale_a": scale_a, "scale_b": scale_b, "tolerance": 1e-3,
                                  "expected": (i * scale_a + i * scale_b).tolist()})
    with open(os.path.join(HERE, "reference_fixtures.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    main()
