"""The IR text this backend is fed is the IR the reference's PPX lowers: pinned on reference-held goldens.

Every recogniser, fusion and GPU test builds its kernels with spoc_b200/sarek_ir.py.  Here that text is printed
as CUDA C by tests/ir_cuda_printer.py, which follows the reference's own printer (sarek-cuda/Sarek_ir_cuda.ml),
and compared byte for byte with the CUDA C the reference generated from the real IR of the same kernels
(tests/golden/generated_cuda/*.cu.txt, copied from benchmarks/descriptions/generated/*_generated.md by
tests/golden/make_generated_cuda.py).  A kernel whose text passes here has the statement structure, the
expression shapes, the parameter order and the names of the reference's IR; the library then has to accept
exactly that text.
"""
import os

import pytest

from spoc_b200 import _lib as L
from spoc_b200 import sarek_ir
from tests import ir_cuda_printer as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "generated_cuda")

CASES = {
    "matrix_mul": (lambda: sarek_ir.matmul_naive_ir(), L.KIND_GEMM_NAIVE),
    "matrix_mul_tiled": (lambda: sarek_ir.matmul_tiled_ir(), L.KIND_GEMM_TILED),
    "vector_add": (lambda: sarek_ir.vector_add_ir(), L.KIND_MAP),
    "stream_triad": (lambda: sarek_ir.stream_triad_ir(), L.KIND_MAP),
    "vector_copy": (lambda: sarek_ir.vector_copy_ir(), L.KIND_MAP),
    "dot_product": (lambda: sarek_ir.block_reduce_ir("dot", name="sarek_kern"), L.KIND_BLOCK_REDUCE),
    "reduction": (lambda: sarek_ir.block_reduce_ir("sum", name="sarek_kern"), L.KIND_BLOCK_REDUCE),
}


def golden(name: str) -> str:
    with open(os.path.join(GOLDEN, name + ".cu.txt")) as f:
        return f.read()


@pytest.mark.parametrize("name", sorted(CASES))
def test_ir_text_prints_as_the_reference_generated_cuda(name):
    build, _ = CASES[name]
    assert P.cuda_source(build()) == golden(name)


@pytest.mark.parametrize("name", sorted(CASES))
def test_library_recognises_the_pinned_ir_text(name):
    """The text that reproduces the reference's rendering is the text sb200_kernel_compile accepts, as the right kind."""
    import ctypes as C
    build, kind = CASES[name]
    lib = L.load()
    h = C.c_uint64(0)
    rc = lib.sb200_kernel_compile(0, build().encode(), b"sarek_kern", C.byref(h))
    assert rc == 0, lib.sb200_last_error_string().decode()
    got = C.c_int(0)
    assert lib.sb200_kernel_kind(h.value, C.byref(got)) == 0
    assert got.value == kind
    lib.sb200_kernel_destroy(h.value)


def test_printer_follows_the_reference_literal_and_operator_rules():
    """Spot checks of printer rules the goldens above do not reach (Sarek_ir_cuda.ml:99-110,210-233)."""
    assert P.expr(["const", "f32", "0.1"]) == "0.10000000000000001f"
    assert P.expr(["const", "f32", "3.0"]) == "3.0f"
    assert P.expr(["const", "f32", "1e+30"]) == "1.0000000000000000e+30f".replace("1.0000000000000000e+30", "%.17g" % 1e30)
    assert P.expr(["const", "i64", "7"]) == "7LL"
    assert P.expr(["unop", "neg", ["evar", "x", "1"]]) == "(-x)"
    assert P.expr(["if", ["binop", "gt", ["evar", "x", "1"], ["const", "f32", "0.0"]], ["evar", "x", "1"], ["const", "f32", "0.0"]]) \
        == "((x > 0.0f) ? x : 0.0f)"
