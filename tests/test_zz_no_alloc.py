"""The allocation-free GEMM entry point, sb200_gemm_f32_noalloc.

Some callers of this library cannot allocate device memory while they run: a
host framework whose caching allocator has already taken all of the GPU's
memory (a further cudaMalloc simply fails), or a caller that keeps other
streams busy and cannot take the device-wide stall of cudaMalloc / cudaFree.
For them the library offers the GEMM with its operand panels in a fixed 32 MiB
device array instead of a grown workspace.  This test drives that entry point
through the C ABI and checks it against the regular sb200_gemm_f32 on the same
inputs, for two calls in a row that differ in shape (so the second call runs
on panels that still hold the first call's contents), then checks that a
problem beyond the fixed array is refused with a clear error.

The file name sorts last on purpose: if it fails under `-x`, every other test
has already run.
"""
import numpy as np
import pytest

from spoc_b200 import _lib as L
from spoc_b200.plugin import _check
from tests import oracle_lib as O
from tests.gpu_util import Dev, dev_from

pytestmark = pytest.mark.gpu


def _both(backend, device, mode, M, N, K, seed):
    lib = L.load()
    a, b, c = O.fill(M * K, seed, 1), O.fill(K * N, seed, 2), O.fill(M * N, seed, 3)
    bias = O.fill(N, seed, 4, kind=1)
    A, B, Cm, Bi = (dev_from(backend, device, x) for x in (a, b, c, bias))
    D_ref, D_new = Dev(backend, device, M * N), Dev(backend, device, M * N)
    try:
        args = (M, N, K, A.ptr, K, B.ptr, N)
        tail = (N, 1.5, Cm.ptr, N, 0.5, Bi.ptr, L.ACT_RELU)
        _check(lib.sb200_gemm_f32(device.id, 0, mode, *args, D_ref.ptr, *tail))
        backend.Device.synchronize(device)
        _check(lib.sb200_gemm_f32_noalloc(device.id, 0, mode, *args, D_new.ptr, *tail))
        want, got = D_ref.download(), D_new.download()
        oracle = O.gemm(a, b, M, N, K, 1.5, 0.5, c, bias, 1).ravel()
        return want, got, oracle
    finally:
        for x in (A, B, Cm, Bi, D_ref, D_new):
            x.free()


@pytest.mark.parametrize("mode", [L.MODE_3XTF32, L.MODE_TF32])
def test_noalloc_gemm_matches_regular_entry_point_twice_in_a_row(backend, device, mode):
    bound = (1e-5 * np.sqrt(520) if mode == L.MODE_3XTF32 else 2e-3) * 1.5 * np.sqrt(2)
    # first call: the larger K, so that the second call's shorter panels overlay stale data
    for (M, N, K, seed) in ((300, 260, 520, 11), (257, 515, 70, 12)):
        want, got, oracle = _both(backend, device, mode, M, N, K, seed)
        # same kernels, same tile schedule: the two entry points agree to the last bit,
        # which is tighter than the tolerance the other GEMM tests allow
        assert O.gemm_rel_error(got, want) <= bound
        assert np.array_equal(got, want)
        assert O.gemm_rel_error(got, oracle) <= bound


def test_noalloc_gemm_rejects_sizes_beyond_its_fixed_scratch(backend, device):
    lib = L.load()
    D = Dev(backend, device, 16)
    try:
        # 4096^3 needs 256 MiB of panels in 3xTF32 mode: far beyond the 32 MiB array
        rc = lib.sb200_gemm_f32_noalloc(device.id, 0, L.MODE_3XTF32, 4096, 4096, 4096, D.ptr, 4096, D.ptr, 4096, D.ptr, 4096,
                                        1.0, 0, 0, 0.0, 0, 0)
        assert rc == L.ERR_TOO_LARGE
        msg = lib.sb200_last_error_string().decode()
        assert "fixed" in msg and "sb200_gemm_f32" in msg
        # degenerate sizes need no scratch at all
        assert lib.sb200_gemm_f32_noalloc(device.id, 0, L.MODE_3XTF32, 0, 8, 8, 0, 8, 0, 8, 0, 8, 1.0, 0, 0, 0.0, 0, 0) == 0
    finally:
        D.free()


def test_noalloc_gemm_checks_operand_extents_like_the_regular_entry_point(backend, device):
    """A result matrix that lies in a library buffer and would run past its end is refused before anything is
    launched, exactly as sb200_gemm_f32 refuses it: a wrong size must not become a memory fault."""
    lib = L.load()
    M, N, K = 64, 64, 64
    A, B = Dev(backend, device, M * K), Dev(backend, device, K * N)
    D_short = Dev(backend, device, M * N - 1024, pad=0)    # the buffer ends 1024 elements before D would
    try:
        rc = lib.sb200_gemm_f32_noalloc(device.id, 0, L.MODE_TF32, M, N, K, A.ptr, K, B.ptr, N, D_short.ptr, N,
                                        1.0, 0, 0, 0.0, 0, 0)
        assert rc == L.ERR_BOUNDS
        assert "GEMM result D" in lib.sb200_last_error_string().decode()
        rc = lib.sb200_gemm_f32(device.id, 0, L.MODE_TF32, M, N, K, A.ptr, K, B.ptr, N, D_short.ptr, N, 1.0, 0, 0, 0.0, 0, 0)
        assert rc == L.ERR_BOUNDS
    finally:
        for x in (A, B, D_short):
            x.free()
