"""ctypes access to the CPU oracle (oracle/native_oracle.c) for the tests.

The oracle is the checker only: nothing under spoc_b200/ imports this.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_f = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_lib = None


def _build() -> str:
    spec = importlib.util.spec_from_file_location("oracle_build", os.path.join(ROOT, "oracle", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_oracle()


def load():
    global _lib
    if _lib is not None:
        return _lib
    lib = C.CDLL(_build())
    i64, f64, i32, vp = C.c_int64, C.c_double, C.c_int, C.c_void_p
    lib.so_fill.argtypes = [_f, i64, C.c_uint64, C.c_uint64, i32, f64, i64]
    lib.so_vector_add.argtypes = [_f, _f, _f, i64]
    lib.so_stream_triad.argtypes = [_f, _f, _f, f64, i64]
    lib.so_chain_triad_square.argtypes = [_f, vp, _f, _f, f64, i64]
    lib.so_matmul_rows.argtypes = [_f, _f, _f, i64, i64, i64, i64, i64, f64, f64, vp, vp, i32]
    lib.so_matmul_points.argtypes = [_f, _f, _f, i64, i64, _i, _i, i64, f64, f64, vp, vp, i32]
    lib.so_matmul_cols.argtypes = [_f, _f, _f, i64, i64, i64, _i, i64, f64, f64, vp, vp, i32]
    lib.so_matmul_tiled.argtypes = [_f, _f, _f, i64, i64, i64]
    lib.so_matmul_naive.argtypes = [_f, _f, _f, i64, i64, i64]
    lib.so_par_vector_add.argtypes = [_f, _f, _f, i64, i32]
    lib.so_par_stream_triad.argtypes = [_f, _f, _f, f64, i64, i32]
    lib.so_par_chain_triad_square.argtypes = [_f, _f, _f, _f, f64, i64, i32]
    lib.so_par_matmul_naive.argtypes = [_f, _f, _f, i64, i64, i64, i64, i64, f64, f64, vp, vp, i32, i32, i32]
    lib.so_par_matmul_tiled.argtypes = [_f, _f, _f, i64, i64, i64, i64, i64, i32]
    lib.so_block_tree_reduce.argtypes = [_f, vp, _f, i64, i64, i32]
    lib.so_block_tree_reduce.restype = None
    lib.so_ulp_distance.argtypes = [C.c_float, C.c_float]
    lib.so_ulp_distance.restype = C.c_int32
    for n in ("so_fill", "so_vector_add", "so_stream_triad", "so_chain_triad_square", "so_matmul_rows", "so_matmul_points",
              "so_matmul_cols", "so_matmul_tiled", "so_matmul_naive", "so_par_vector_add", "so_par_stream_triad",
              "so_par_chain_triad_square", "so_par_matmul_naive", "so_par_matmul_tiled"):
        getattr(lib, n).restype = None
    _lib = lib
    return lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def fill(n: int, seed: int, stream: int, kind: int = 0, sigma: float = 1.0, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    load().so_fill(out, n, seed, stream, kind, sigma, first)
    return out


def gemm(a, b, m, n, k, alpha=1.0, beta=0.0, cin=None, bias=None, act=0, r0=0, r1=None) -> np.ndarray:
    """Rows [r0, r1) of act(alpha*A.B + beta*C + bias) under Native semantics."""
    r1 = m if r1 is None else r1
    out = np.empty((r1 - r0) * n, dtype=np.float32)
    load().so_matmul_rows(a, b, out, m, n, k, r0, r1, alpha, beta, _ptr(cin), _ptr(bias), act)
    return out.reshape(r1 - r0, n)


def gemm_points(a, b, n, k, rows, cols, alpha=1.0, beta=0.0, cin=None, bias=None, act=0) -> np.ndarray:
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    cols = np.ascontiguousarray(cols, dtype=np.int64)
    out = np.empty(len(rows), dtype=np.float32)
    load().so_matmul_points(a, b, out, n, k, rows, cols, len(rows), alpha, beta, _ptr(cin), _ptr(bias), act)
    return out


def gemm_cols(a, b, m, n, k, cols, alpha=1.0, beta=0.0, cin=None, bias=None, act=0) -> np.ndarray:
    cols = np.ascontiguousarray(cols, dtype=np.int64)
    out = np.empty(m * len(cols), dtype=np.float32)
    load().so_matmul_cols(a, b, out, m, n, k, cols, len(cols), alpha, beta, _ptr(cin), _ptr(bias), act)
    return out.reshape(m, len(cols))


def ulp_distance(x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """Integer distance between float32 bit patterns on the ordered-integer line."""
    ix = x.view(np.int32).astype(np.int64)
    iy = y.view(np.int32).astype(np.int64)
    ix = np.where(ix < 0, -(2 ** 31) - ix, ix)
    iy = np.where(iy < 0, -(2 ** 31) - iy, iy)
    return np.abs(ix - iy)


def gemm_rel_error(got: np.ndarray, ref: np.ndarray) -> float:
    """max |got-ref| / max(|ref|, rms(ref)): relative error with the root mean
    square of the reference as floor, so entries near zero of a zero-mean
    product do not dominate."""
    ref64 = ref.astype(np.float64)
    rho = float(np.sqrt(np.mean(ref64 * ref64))) if ref.size else 0.0
    den = np.maximum(np.abs(ref64), rho if rho > 0 else 1.0)
    return float(np.max(np.abs(got.astype(np.float64) - ref64) / den)) if ref.size else 0.0
