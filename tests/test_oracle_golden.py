"""The CPU oracle against the reference's own fixtures for this path, and its internal consistency.

The fixtures (tests/golden/reference_fixtures.json, made by tests/golden/make_golden.py) are the closed
forms the reference's tests and benchmarks verify against, with the reference's tolerances.
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

from tests import oracle_lib as O

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_fixtures.json")))


@pytest.mark.parametrize("case", GOLDEN["matmul"], ids=lambda c: f"{c['m']}x{c['n']}x{c['k']}")
def test_matmul_fixture(case):
    m, n, k = case["m"], case["n"], case["k"]
    a = ((np.arange(m * k) % 10) / 10.0).astype(np.float32)   # Vector.set narrows to float32
    b = (((np.arange(k * n) + 1) % 10) / 10.0).astype(np.float32)
    exp = np.array(case["expected"]).reshape(m, n)
    lib = O.load()
    naive, tiled = np.empty(m * n, np.float32), np.empty(m * n, np.float32)
    lib.so_matmul_naive(a, b, naive, m, n, k)
    lib.so_matmul_tiled(a, b, tiled, m, n, k)
    rows = O.gemm(a, b, m, n, k)
    assert np.max(np.abs(naive.reshape(m, n) - exp)) <= case["tolerance"]
    # naive, tiled (with zero-padded ragged tiles) and the row form sum k ascending: bit-identical
    assert np.array_equal(naive, tiled)
    assert np.array_equal(naive.reshape(m, n), rows)


def test_triad_fixture():
    t = GOLDEN["triad"]
    n = t["n"]
    i = np.arange(n)
    b, c = ((i % 100) / 100.0).astype(np.float32), (((i + 1) % 100) / 100.0).astype(np.float32)
    a = np.empty(n, np.float32)
    O.load().so_stream_triad(a, b, c, t["scalar"], n)
    assert np.max(np.abs(a - np.array(t["expected"]))) <= t["tolerance"]


@pytest.mark.parametrize("case", GOLDEN["vector_add"], ids=lambda c: f"scale{c['scale_a']}")
def test_vector_add_fixture(case):
    n = case["n"]
    i = np.arange(n, dtype=np.float64)
    a, b = (i * case["scale_a"]).astype(np.float32), (i * case["scale_b"]).astype(np.float32)
    c = np.empty(n, np.float32)
    O.load().so_vector_add(a, b, c, n)
    assert np.max(np.abs(c - np.array(case["expected"]))) <= case["tolerance"]


def test_native_rounding_rules():
    """One rounding at the store, double arithmetic in between (the rules at the top of native_oracle.c)."""
    lib = O.load()
    rng = np.random.default_rng(0)
    n = 100000
    b, c = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    a = np.empty(n, np.float32)
    lib.so_stream_triad(a, b, c, 3.0, n)
    want = (b.astype(np.float64) + c.astype(np.float64) * 3.0).astype(np.float32)
    assert np.array_equal(a, want)
    # differs from per-operation float32 rounding somewhere: the Interpreter backend's semantics are not Native's
    per_op = (b + (c * np.float32(3.0)).astype(np.float32)).astype(np.float32)
    assert not np.array_equal(a, per_op)
    # the chain stores (and rounds) the intermediate, as two Native launches do
    d, a_tmp = np.empty(n, np.float32), np.empty(n, np.float32)
    lib.so_chain_triad_square(d, a_tmp.ctypes.data_as(C.c_void_p), b, c, 3.0, n)
    assert np.array_equal(a_tmp, want)
    want_d = (want.astype(np.float64) * want.astype(np.float64) + b.astype(np.float64)).astype(np.float32)
    assert np.array_equal(d, want_d)


def test_gemm_epilogue_and_samplers_agree():
    m, n, k = 37, 53, 41
    a, b, c = O.fill(m * k, 9, 1), O.fill(k * n, 9, 2), O.fill(m * n, 9, 3)
    bias = O.fill(n, 9, 4, kind=1)
    full = O.gemm(a, b, m, n, k, 1.5, 0.5, c, bias, 1)
    a64, b64 = a.reshape(m, k).astype(np.float64), b.reshape(k, n).astype(np.float64)
    acc = np.zeros((m, n))
    for i in range(k):                      # same order: k ascending, one accumulator
        acc = acc + np.outer(a64[:, i], b64[i])
    want = np.maximum(1.5 * acc + 0.5 * c.reshape(m, n).astype(np.float64) + bias.astype(np.float64), 0.0).astype(np.float32)
    assert np.array_equal(full, want)
    cols = [0, 7, n - 1]
    assert np.array_equal(O.gemm_cols(a, b, m, n, k, cols, 1.5, 0.5, c, bias, 1), full[:, cols])
    rows, cs = np.array([0, 5, m - 1]), np.array([n - 1, 3, 0])
    assert np.array_equal(O.gemm_points(a, b, n, k, rows, cs, 1.5, 0.5, c, bias, 1), full[rows, cs])
    assert np.array_equal(O.gemm(a, b, m, n, k, 1.5, 0.5, c, bias, 1, r0=5, r1=9), full[5:9])


def test_parallel_partition_matches_serial():
    lib = O.load()
    n = 10007
    b, c = O.fill(n, 3, 2), O.fill(n, 3, 3)
    s, p = np.empty(n, np.float32), np.empty(n, np.float32)
    lib.so_stream_triad(s, b, c, 3.0, n)
    lib.so_par_stream_triad(p, b, c, 3.0, n, 3)
    assert np.array_equal(s, p)
    lib.so_vector_add(b, c, s, n)
    lib.so_par_vector_add(b, c, p, n, 4)
    assert np.array_equal(s, p)
    d1, a1, d2 = np.empty(n, np.float32), np.empty(n, np.float32), np.empty(n, np.float32)
    lib.so_par_chain_triad_square(d1, a1, b, c, 3.0, n, 3)
    lib.so_chain_triad_square(d2, None, b, c, 3.0, n)
    assert np.array_equal(d1, d2)
    m, nn, k = 50, 70, 30
    a, bb = O.fill(m * k, 4, 1), O.fill(k * nn, 4, 2)
    ser = O.gemm(a, bb, m, nn, k).ravel()
    par = np.zeros(m * nn, np.float32)
    lib.so_par_matmul_naive(a, bb, par, m, nn, k, 0, m * nn, 1.0, 0.0, None, None, 0, 0, 4)
    assert np.array_equal(ser, par)
    part = np.zeros(m * nn, np.float32)
    lib.so_par_matmul_naive(a, bb, part, m, nn, k, 700, 1500, 1.0, 0.0, None, None, 0, 0, 2)
    assert np.array_equal(part[700:1500], ser[700:1500]) and not part[:700].any() and not part[1500:].any()
    til = np.zeros(m * nn, np.float32)
    lib.so_par_matmul_tiled(a, bb, til, m, nn, k, 0, 0, 3)
    assert np.array_equal(ser, til)


def test_generator_is_the_documented_function():
    def splitmix(x):
        x = (x + 0x9E3779B97F4A7C15) & (2 ** 64 - 1)
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
        return x ^ (x >> 31)
    seed, stream = 20260101, 2
    got = O.fill(64, seed, stream, first=1000)
    for j in range(64):
        u = splitmix(seed ^ ((stream * 0x9E3779B97F4A7C15) & (2 ** 64 - 1)) ^ (1000 + j)) >> 40
        assert got[j] == np.float32(u / 8388608.0 - 1.0)
    assert np.all(np.abs(O.fill(10000, 1, 4, kind=1)) <= 0.1)
    z = O.fill(200000, 1, 1, kind=2, sigma=2.0)
    assert abs(z.mean()) < 0.02 and abs(z.std() - 2.0) < 0.02
    assert np.array_equal(O.fill(100, 5, 1, first=50), O.fill(150, 5, 1)[50:])


def test_ulp_distance_helper():
    x = np.array([1.0, -1.0, 0.0, 1.0], np.float32)
    y = np.array([np.nextafter(np.float32(1.0), np.float32(2.0)), -1.0, -0.0, 1.5], np.float32)
    d = O.ulp_distance(x, y)
    assert d[0] == 1 and d[1] == 0 and d[2] == 0 and d[3] > 1000


def test_block_tree_reduce_matches_reference_fixture():
    """benchmarks/bench_dot_product.ml:58-66: a=(i mod 100)/100, b=((i+1) mod 100)/100, expected = sequential
    double sum of a*b; the benchmark sums the per-block partial results on the host."""
    n, block = 100000, 256
    i = np.arange(n)
    a64, b64 = (i % 100) / 100.0, ((i + 1) % 100) / 100.0
    a, b = a64.astype(np.float32), b64.astype(np.float32)
    nblocks = (n + block - 1) // block
    out = np.empty(nblocks, np.float32)
    O.load().so_block_tree_reduce(a, b.ctypes.data_as(C.c_void_p), out, n, nblocks, block)
    expected = float(np.sum(a64 * b64))
    assert abs(float(out.astype(np.float64).sum()) - expected) / expected < 1e-5
    # per block: the tree order in double, against an independent numpy evaluation of the same tree
    prod = np.zeros(nblocks * block)
    prod[:n] = a.astype(np.float64) * b.astype(np.float64)
    t = prod.reshape(nblocks, block)
    c = block // 2
    while c >= 1:
        t = t[:, :c] + t[:, c:2 * c]
        c //= 2
    assert np.array_equal(out, t[:, 0].astype(np.float32))
