"""Staged copies between pageable host memory and the device (the transfer path around the kernels,
sarek/core/Transfer.ml:229-322): same bytes as the plain copy, same ordering guarantees."""
import ctypes as C

import numpy as np
import pytest

from spoc_b200 import Vector
from spoc_b200 import _lib as L
from spoc_b200.plugin import _check
from tests import oracle_lib as O

pytestmark = pytest.mark.gpu

MIB = 1 << 20


@pytest.mark.parametrize("nbytes", [16 * MIB, 16 * MIB + 4, 20 * MIB - 4, 64 * MIB + 4 * 12345, 4 * MIB * 9 + 8])
def test_staged_copies_move_the_same_bytes_as_plain_copies(backend, device, nbytes):
    lib = L.load()
    n = nbytes // 4
    rng = np.random.default_rng(nbytes)
    src = rng.integers(0, 2 ** 32, size=n, dtype=np.uint32)          # pageable, every bit pattern
    buf = backend.Memory.alloc(device, n, np.float32)
    pinned = C.c_void_p()
    _check(lib.sb200_host_alloc(nbytes, C.byref(pinned)))
    try:
        _check(lib.sb200_memcpy_htod(device.id, buf.ptr, src.ctypes.data, nbytes))          # staged up
        _check(lib.sb200_memcpy_dtoh(device.id, pinned, buf.ptr, nbytes))                    # plain down (pinned)
        via_pinned = np.frombuffer((C.c_char * nbytes).from_address(pinned.value), dtype=np.uint32)
        assert np.array_equal(via_pinned, src)
        back = np.zeros(n, dtype=np.uint32)
        _check(lib.sb200_memcpy_dtoh(device.id, back.ctypes.data, buf.ptr, nbytes))         # staged down
        assert np.array_equal(back, src)
        # plain up from pinned memory, staged down again
        rev = np.ascontiguousarray(src[::-1])          # kept alive while its address is in use
        C.memmove(pinned, rev.ctypes.data, nbytes)
        _check(lib.sb200_memcpy_htod(device.id, buf.ptr, pinned, nbytes))
        _check(lib.sb200_memcpy_dtoh(device.id, back.ctypes.data, buf.ptr, nbytes))
        assert np.array_equal(back, rev)
    finally:
        _check(lib.sb200_host_free(pinned))
        backend.Memory.free(buf)


def test_staged_copy_is_ordered_after_earlier_launches(backend, device):
    """A download straight after an asynchronous launch returns what the launch wrote, as the plain
    synchronous copy does."""
    lib = L.load()
    n = 24 * MIB // 4
    buf = backend.Memory.alloc(device, n, np.float32)
    try:
        _check(lib.sb200_memset32(device.id, buf.ptr, 0, n, 0))
        _check(lib.sb200_fill_f32(device.id, 0, buf.ptr, n, 77, 1, 0, 1.0, 0))     # asynchronous
        got = np.empty(n, np.float32)
        _check(lib.sb200_memcpy_dtoh(device.id, got.ctypes.data, buf.ptr, 4 * n))
        assert np.array_equal(got, O.fill(n, 77, 1))
        # and an upload followed by a kernel that reads the buffer
        host = O.fill(n, 78, 2)
        _check(lib.sb200_memcpy_htod(device.id, buf.ptr, host.ctypes.data, 4 * n))
        out = backend.Memory.alloc(device, n, np.float32)
        _check(lib.sb200_vector_add_f32(device.id, 0, out.ptr, buf.ptr, buf.ptr, n))
        _check(lib.sb200_memcpy_dtoh(device.id, got.ctypes.data, out.ptr, 4 * n))
        assert np.array_equal(got, host + host)
        backend.Memory.free(out)
    finally:
        backend.Memory.free(buf)


def test_large_vector_round_trip_through_the_host_mirror(backend, device):
    n = 40 * MIB // 4 + 3
    data = O.fill(n, 5, 1)
    v = Vector(backend, data.copy())
    v.to_device(device)
    v.location = Vector.STALE_CPU
    v.host[:] = 0
    assert np.array_equal(v.to_array(), data)
    v.free()


def test_vector_is_pinned_in_place_on_its_second_large_transfer(backend, device):
    """A Vector owns its host array, so the plugin registers it with the driver once it is moved a second time; results
    are unchanged, the registration goes away with free(), and small vectors are left alone."""
    from spoc_b200 import Vector
    n = (16 << 20) // 4
    big, small = Vector(backend, np.arange(n, dtype=np.float32)), Vector(backend, np.arange(1000, dtype=np.float32))
    try:
        for v in (big, small):
            v.to_device(device)
            assert not v._pinned
            v.location = Vector.STALE_CPU     # as after a launch: the next host read downloads
            v.host[:] = -1.0
            got = v.to_array()
            assert got[0] == 0.0 and got[-1] == np.float32(len(got) - 1)
        assert big._pinned and not small._pinned
        big.location = Vector.CPU
        big.host[:] = 7.0
        big.to_device(device)                 # third transfer: from registered memory
        big.location = Vector.STALE_CPU
        big.host[:] = 0.0
        assert np.all(big.to_array() == 7.0)
    finally:
        big.free()
        small.free()
    assert not big._pinned
