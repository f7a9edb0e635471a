"""The CPU oracle computes what the pinned IR says, under the Native backend's rounding rules.

tests/ir_interp.py executes a kernel's IR text thread by thread.  Under the "native" discipline (double operations, one
rounding per vector store) its results must equal the oracle's (oracle/native_oracle.c) bit for bit, for every kernel of the
path, on the very IR text that tests/test_ir_golden.py pins on the reference's generated code.  Under the "interpreter"
discipline (every float32 operation rounds, sarek/sarek/Sarek_ir_interp.ml:175-211) the results must differ — slightly —
which shows that the comparison can tell the two semantics apart.
"""
import ctypes as C

import numpy as np
import pytest

from spoc_b200 import sarek_ir
from tests import oracle_lib as O
from tests.ir_interp import run_kernel

EPI = dict(alpha=1.5, beta=0.5, c="c", bias="bias", relu=True)


def _matmul_case(m, n, k, seed, epilogue):
    a, b, c = O.fill(m * k, seed, 1), O.fill(k * n, seed, 2), O.fill(m * n, seed, 3)
    bias = O.fill(n, seed, 4, kind=1)
    ref = O.gemm(a, b, m, n, k, 1.5, 0.5, c, bias, 1) if epilogue else O.gemm(a, b, m, n, k)
    return a, b, c, bias, ref.ravel()


@pytest.mark.parametrize("shape", ["naive", "tiled"])
@pytest.mark.parametrize("epilogue", [False, True], ids=["plain", "epilogue"])
def test_matmul_ir_under_native_rules_equals_the_oracle_bit_for_bit(shape, epilogue):
    m, n, k = 21, 19, 37
    a, b, c, bias, ref = _matmul_case(m, n, k, 5, epilogue)
    out = np.full(m * n, -7.0, np.float32)
    vecs = {"a": a, "b": b, "c": c.copy(), "bias": bias, "d": out} if epilogue else {"a": a, "b": b, "c": out}
    epi = EPI if epilogue else None
    if shape == "naive":
        run_kernel(sarek_ir.matmul_naive_ir(epilogue=epi), vecs, {"m": m, "n": n, "k": k}, grid=((m * n + 63) // 64,), block=(64,))
    else:
        run_kernel(sarek_ir.matmul_tiled_ir(epilogue=epi), vecs, {"m": m, "n": n, "k": k}, grid=((n + 15) // 16, (m + 15) // 16),
                   block=(16, 16))
    assert np.array_equal(out, ref)


def test_matmul_ir_under_interpreter_rules_differs_slightly():
    m, n, k = 16, 16, 96
    a, b, _, _, ref = _matmul_case(m, n, k, 6, False)
    out = np.zeros(m * n, np.float32)
    run_kernel(sarek_ir.matmul_naive_ir(), {"a": a, "b": b, "c": out}, {"m": m, "n": n, "k": k}, grid=(m * n // 64,), block=(64,),
               discipline="interpreter")
    d = O.ulp_distance(out, ref)
    assert d.max() >= 1, "per-operation rounding must show against one rounding at the store"
    assert np.max(np.abs(out.astype(np.float64) - ref) / np.sqrt(np.mean(ref.astype(np.float64) ** 2))) < 1e-5


def test_map_kernels_under_native_rules_equal_the_oracle_bit_for_bit():
    n = 1000
    lib = O.load()
    b, c = O.fill(n, 7, 2), O.fill(n, 7, 3)
    grid, block = ((n + 63) // 64,), (64,)
    # vector_add
    out, ref = np.zeros(n, np.float32), np.empty(n, np.float32)
    run_kernel(sarek_ir.vector_add_ir(), {"a": b, "b": c, "c": out}, {"n": n}, grid, block)
    lib.so_vector_add(b, c, ref, n)
    assert np.array_equal(out, ref)
    # stream_triad, then the guarded consumer d = a*a + b: the unfused chain, as Native runs it
    a_out, d_out = np.zeros(n, np.float32), np.zeros(n, np.float32)
    run_kernel(sarek_ir.stream_triad_ir(), {"a": a_out, "b": b, "c": c}, {"scalar": 3.0, "n": n}, grid, block)
    run_kernel(sarek_ir.square_add_guarded_ir(), {"d": d_out, "a": a_out, "b": b}, {"n": n}, grid, block)
    ref_d, ref_a = np.empty(n, np.float32), np.empty(n, np.float32)
    lib.so_chain_triad_square(ref_d, ref_a.ctypes.data_as(C.c_void_p), b, c, 3.0, n)
    assert np.array_equal(a_out, ref_a) and np.array_equal(d_out, ref_d)
    # the launch covers fewer threads than elements: the rest stays untouched
    part = np.full(n, -1.0, np.float32)
    run_kernel(sarek_ir.vector_add_ir(), {"a": b, "b": c, "c": part}, {"n": n}, (3,), (64,))
    assert np.array_equal(part[:192], ref[:192]) and np.all(part[192:] == -1.0)
    # vector_copy
    cp = np.zeros(n, np.float32)
    run_kernel(sarek_ir.vector_copy_ir(), {"a": b, "b": cp}, {"n": n}, grid, block)
    assert np.array_equal(cp, b)


def test_triad_under_interpreter_rules_differs_from_native_somewhere():
    n = 4096
    b, c = O.fill(n, 8, 2), O.fill(n, 8, 3)
    nat, itp = np.zeros(n, np.float32), np.zeros(n, np.float32)
    run_kernel(sarek_ir.stream_triad_ir(), {"a": nat, "b": b, "c": c}, {"scalar": 3.0, "n": n}, (n // 64,), (64,))
    run_kernel(sarek_ir.stream_triad_ir(), {"a": itp, "b": b, "c": c}, {"scalar": 3.0, "n": n}, (n // 64,), (64,), discipline="interpreter")
    d = O.ulp_distance(nat, itp)
    assert 0 < (d > 0).sum() < n // 2 and d.max() <= 1


@pytest.mark.parametrize("kind", ["dot", "sum"])
def test_block_tree_reductions_under_native_rules_equal_the_oracle_bit_for_bit(kind):
    block, nblocks = 64, 5
    n = block * nblocks - 17           # the last block is ragged: the load superstep writes 0.0 past n
    lib = O.load()
    a, b = O.fill(n, 9, 1), O.fill(n, 9, 2)
    out, ref = np.zeros(nblocks, np.float32), np.empty(nblocks, np.float32)
    ir = sarek_ir.block_reduce_ir(kind, block)
    vecs = {"a": a, "b": b, "output": out} if kind == "dot" else {"input": a, "output": out}
    run_kernel(ir, vecs, {"n": n}, (nblocks,), (block,))
    lib.so_block_tree_reduce(a, b.ctypes.data_as(C.c_void_p) if kind == "dot" else None, ref, n, nblocks, block)
    assert np.array_equal(out, ref)
