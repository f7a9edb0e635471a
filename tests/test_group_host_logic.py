"""Host-side behaviour of the device-group entry points that needs no GPU: argument errors are reported before any
GPU work, the row split is the reference's partition rule, and a machine without a usable GPU gets a clear error
instead of a fallback."""
import ctypes as C

import pytest

from spoc_b200 import _lib as L
from spoc_b200.sharding import partition


def test_row_block_is_the_reference_partition_rule():
    lib = L.load()
    for total, parts in ((10, 3), (8, 4), (2, 4), (0, 2), (65536, 8), (32769, 8), (7, 1)):
        want = partition(total, parts)
        for i in range(parts):
            first, count = C.c_int64(-1), C.c_int64(-1)
            assert lib.sb200_row_block(total, parts, i, C.byref(first), C.byref(count)) == 0
            assert (first.value, count.value) == want[i]
    first, count = C.c_int64(0), C.c_int64(0)
    assert lib.sb200_row_block(10, 0, 0, C.byref(first), C.byref(count)) == L.ERR_INVALID_VALUE
    assert lib.sb200_row_block(10, 3, 3, C.byref(first), C.byref(count)) == L.ERR_INVALID_VALUE
    assert lib.sb200_row_block(-1, 3, 0, C.byref(first), C.byref(count)) == L.ERR_INVALID_VALUE


@pytest.mark.parametrize("ngpus", [0, -1, 9])
def test_group_size_out_of_range_is_refused_before_anything_else(ngpus):
    lib = L.load()
    h = C.c_uint64(123)
    assert lib.sb200_group_create(ngpus, None, C.byref(h)) == L.ERR_INVALID_VALUE
    assert h.value == 0
    assert "between 1 and 8" in lib.sb200_last_error_string().decode()


def test_group_calls_on_unknown_handles_fail_cleanly():
    lib = L.load()
    n = C.c_int(0)
    ms = C.c_float(0)
    assert lib.sb200_group_size(0xdead, C.byref(n)) == L.ERR_INVALID_HANDLE
    assert lib.sb200_group_last_ms(0xdead, C.byref(ms)) == L.ERR_INVALID_HANDLE
    assert lib.sb200_group_destroy(0xdead) == L.ERR_INVALID_HANDLE
    assert lib.sb200_group_destroy(0) == 0
    tab = (C.c_uint64 * 1)(0)
    assert lib.sb200_gemm_sharded(0xdead, L.MODE_TF32, 8, 8, 8, tab, 8, 0, 8, tab, 8, 1.0, None, 8, 0.0, 0, 0, 0) == L.ERR_INVALID_HANDLE
    assert lib.sb200_gemm_sharded_host(0xdead, L.MODE_TF32, 8, 8, 8, None, 8, None, 8, None, 8, 1.0, None, 8, 0.0, None, 0) \
        == L.ERR_INVALID_HANDLE


def test_group_without_a_usable_gpu_reports_no_device():
    lib = L.load()
    cnt = C.c_int(0)
    lib.sb200_device_count(C.byref(cnt))
    if cnt.value > 0:
        pytest.skip("a GPU is present; the no-device answer is what a CPU-only box gives")
    h = C.c_uint64(0)
    assert lib.sb200_group_create(1, None, C.byref(h)) == L.ERR_NO_DEVICE
    assert h.value == 0
