"""The device-group entry points on real GPUs.

A group of one GPU must behave exactly as the per-device operator (bit for bit, every gather flag); argument
errors that need the device count are reported with nothing launched; the host-operand form matches the oracle.
The tests that need two GPUs check every multi-GPU form against the single-GPU result bit for bit and skip on a
one-GPU machine.
"""
import ctypes as C
import math

import numpy as np
import pytest

from spoc_b200 import _lib as L
from spoc_b200.plugin import _check
from spoc_b200.sharding import DeviceGroup, partition
from tests import oracle_lib as O
from tests.gpu_util import CANARY, Dev, dev_from, gemm

pytestmark = pytest.mark.gpu
MODES = [L.MODE_3XTF32, L.MODE_TF32, L.MODE_3XF16, L.MODE_F16, L.MODE_3XMIXED]


def _tol(mode, K):
    return (max(1e-5 * math.sqrt(K), 1e-6) if mode in (L.MODE_3XTF32, L.MODE_3XF16, L.MODE_3XMIXED) else 2e-3) * 1.5 * math.sqrt(2)


@pytest.fixture(autouse=True)
def mixed_mode_on_small_products():
    """The mixed mode takes products from 2^34 multiply-adds by default; lowered here so that its own kernels run."""
    L.load().sb200_set_mixed_min_macs(1 << 20)
    yield
    L.load().sb200_set_mixed_min_macs(0)


def _same(mode, got, want):
    """Row blocks reproduce the one-launch product bit for bit — except in the mixed mode, whose fp16 panel scales follow
    the largest magnitude of the rows a call sees and which hands row blocks below its size threshold to 3xTF32: there
    the forms agree far inside the mode's error bound (1e-5 of the result's rms; TF32 mode would be at 1e-3)."""
    got, want = np.asarray(got), np.asarray(want)
    if mode != L.MODE_3XMIXED:
        return np.array_equal(got, want)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    return float(np.abs(got.astype(np.float64) - want).max()) <= 1e-5 * max(rms, 1e-30)


def _problem(M, N, K, seed):
    return O.fill(M * K, seed, 1), O.fill(K * N, seed, 2), O.fill(M * N, seed, 3), O.fill(N, seed, 4, kind=1)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("gather", [DeviceGroup.GATHER_NONE, DeviceGroup.GATHER_FUSED, DeviceGroup.GATHER_NCCL])
def test_group_of_one_equals_the_per_device_operator(backend, device, mode, gather):
    M, N, K = 389, 516, 200
    a, b, c, bias = _problem(M, N, K, 81)
    A, B, Cm, Bi = (dev_from(backend, device, x) for x in (a, b, c, bias))
    D0, D1 = Dev(backend, device, M * N), Dev(backend, device, M * N)
    grp = DeviceGroup([device.id])
    try:
        gemm(backend, device, mode, M, N, K, A, B, D0, alpha=1.5, C_=Cm, beta=0.5, bias=Bi, act=1)
        ms = grp.gemm(mode, M, N, K, [A.ptr], B.ptr, [D1.ptr], alpha=1.5, c_shards=[Cm.ptr], beta=0.5, bias=Bi.ptr, act=1, gather=gather)
        assert ms > 0.0
        assert np.array_equal(D0.download(), D1.download())
        # the same call again with "B resident": nothing to replicate in a group of one, same result
        D1.clear()
        grp.gemm(mode, M, N, K, [A.ptr], B.ptr, [D1.ptr], alpha=1.5, c_shards=[Cm.ptr], beta=0.5, bias=Bi.ptr, act=1, gather=gather,
                 b_resident=True)
        assert np.array_equal(D0.download(), D1.download())
        assert grp.row_block(M, 0) == (0, M)
    finally:
        grp.close()
        for x in (A, B, Cm, Bi, D0, D1):
            x.free()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("pinned", [False, True])
def test_group_of_one_host_operands_match_the_oracle(backend, device, mode, pinned):
    lib = L.load()
    M, N, K = 1100, 520, 136        # more than four 256-row chunks' worth of rows: every chunk path runs
    a, b, c, bias = _problem(M, N, K, 82)
    d = np.full(M * N, CANARY, np.float32)
    held = []
    if pinned:
        def pin(x):
            p = C.c_void_p()
            _check(lib.sb200_host_alloc(x.nbytes, C.byref(p)))
            held.append(p)
            v = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(x.size,))
            v[:] = x
            return v
        a, b, c, d = pin(a), pin(b), pin(c), pin(d)
    grp = DeviceGroup([device.id])
    try:
        grp.gemm_host(mode, M, N, K, a, b, d, alpha=1.5, c=c, beta=0.5, bias=bias, act=1)
        ref = O.gemm(np.array(a), np.array(b), M, N, K, 1.5, 0.5, np.array(c), bias, 1)
        assert O.gemm_rel_error(np.array(d).reshape(M, N), ref) <= _tol(mode, K)
        # and equal to the single-GPU host call bit for bit
        d2 = np.empty(M * N, np.float32)
        _check(lib.sb200_gemm_f32_host(device.id, mode, M, N, K, a.ctypes.data, K, b.ctypes.data, N, d2.ctypes.data, N, 1.5,
                                       c.ctypes.data, N, 0.5, bias.ctypes.data, 1))
        assert _same(mode, np.array(d), d2)
    finally:
        grp.close()
        for p in held:
            _check(lib.sb200_host_free(p))


def test_group_argument_errors_launch_nothing(backend, device):
    lib = L.load()
    before = backend.launch_count()
    h = C.c_uint64(0)
    count = backend.Device.count()
    devs = (C.c_int * 2)(0, count)            # second member does not exist
    assert lib.sb200_group_create(2, devs, C.byref(h)) == L.ERR_INVALID_VALUE and h.value == 0
    assert "usable" in lib.sb200_last_error_string().decode()
    devs = (C.c_int * 2)(0, 0)                # the same GPU twice
    assert lib.sb200_group_create(2, devs, C.byref(h)) == L.ERR_INVALID_VALUE and h.value == 0
    grp = DeviceGroup([device.id])
    try:
        tab = (C.c_uint64 * 1)(0)
        rc = lib.sb200_gemm_sharded(grp.handle, L.MODE_TF32, 8, 8, 8, tab, 8, 0, 8, tab, 8, 1.0, None, 8, 0.0, 0, 0, 3)
        assert rc == L.ERR_INVALID_VALUE      # both gather flags
        rc = lib.sb200_gemm_sharded(grp.handle, L.MODE_TF32, 8, 8, 8, tab, 8, 0, 8, tab, 8, 1.0, None, 8, 0.0, 0, 0, 64)
        assert rc == L.ERR_INVALID_VALUE      # unknown flag
        rc = lib.sb200_gemm_sharded(grp.handle, L.MODE_TF32, 8, 8, 8, tab, 8, 0, 8, tab, 8, 1.0, None, 8, 0.0, 0, 0, 0)
        assert rc == L.ERR_INVALID_VALUE      # null shard pointers
    finally:
        grp.close()
    assert backend.launch_count() == before


def _two_gpus(backend):
    if backend.Device.count() < 2:
        pytest.skip("needs two GPUs")
    return backend.Device.get(0), backend.Device.get(1)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("M", [1024, 777])
def test_two_gpu_group_every_form_equals_one_gpu(backend, mode, M):
    """Row blocks, the gather fused into the epilogue and the NCCL gather on two GPUs, against the single-GPU result
    bit for bit; M = 777 gives unequal blocks (389 + 388), which the NCCL gather serves with one broadcast per block."""
    d0, d1 = _two_gpus(backend)
    N, K = 520, 264
    a, b, c, bias = _problem(M, N, K, 83)
    parts = partition(M, 2)
    devs = (d0, d1)
    A = [dev_from(backend, dv, a[f * K:(f + r) * K]) for dv, (f, r) in zip(devs, parts)]
    Cs = [dev_from(backend, dv, c[f * N:(f + r) * N]) for dv, (f, r) in zip(devs, parts)]
    B, Bi = dev_from(backend, d0, b), dev_from(backend, d0, bias)
    Afull, Cfull, Dref = dev_from(backend, d0, a), dev_from(backend, d0, c), Dev(backend, d0, M * N)
    blocks = [Dev(backend, dv, r * N) for dv, (f, r) in zip(devs, parts)]
    full = [Dev(backend, dv, M * N) for dv in devs]
    grp = DeviceGroup([d0.id, d1.id])
    try:
        backend.Device.set_current(d0)
        gemm(backend, d0, mode, M, N, K, Afull, B, Dref, alpha=1.5, C_=Cfull, beta=0.5, bias=Bi, act=1)
        want = Dref.download().reshape(M, N)
        kw = dict(alpha=1.5, c_shards=[x.ptr for x in Cs], beta=0.5, bias=Bi.ptr, act=1)
        grp.gemm(mode, M, N, K, [x.ptr for x in A], B.ptr, [x.ptr for x in blocks], **kw)
        for blk, (f, r) in zip(blocks, parts):
            assert _same(mode, blk.download().reshape(r, N), want[f:f + r])
        for gather in (DeviceGroup.GATHER_FUSED, DeviceGroup.GATHER_NCCL):
            for x in full:
                x.clear()
            ms = grp.gemm(mode, M, N, K, [x.ptr for x in A], B.ptr, [x.ptr for x in full], gather=gather,
                          b_resident=(gather == DeviceGroup.GATHER_NCCL), **kw)
            assert ms > 0
            for x in full:
                assert _same(mode, x.download().reshape(M, N), want)
        ref = O.gemm(a, b, M, N, K, 1.5, 0.5, c, bias, 1)
        assert O.gemm_rel_error(want, ref) <= _tol(mode, K)
    finally:
        grp.close()
        for x in A + Cs + [B, Bi, Afull, Cfull, Dref] + blocks + full:
            x.free()
        backend.Device.set_current(d0)


@pytest.mark.parametrize("mode", MODES)
def test_two_gpu_group_host_operands(backend, mode):
    d0, d1 = _two_gpus(backend)
    lib = L.load()
    M, N, K = 2101, 520, 136
    a, b, c, bias = _problem(M, N, K, 84)
    d = np.full(M * N, CANARY, np.float32)
    grp = DeviceGroup([d0.id, d1.id])
    try:
        grp.gemm_host(mode, M, N, K, a, b, d, alpha=1.5, c=c, beta=0.5, bias=bias, act=1)
        d1gpu = np.empty(M * N, np.float32)
        _check(lib.sb200_gemm_f32_host(d0.id, mode, M, N, K, a.ctypes.data, K, b.ctypes.data, N, d1gpu.ctypes.data, N, 1.5,
                                       c.ctypes.data, N, 0.5, bias.ctypes.data, 1))
        assert _same(mode, d, d1gpu)
        ref = O.gemm(a, b, M, N, K, 1.5, 0.5, c, bias, 1)
        assert O.gemm_rel_error(d.reshape(M, N), ref) <= _tol(mode, K)
    finally:
        grp.close()
        backend.Device.set_current(d0)


@pytest.mark.parametrize("gpus", [1, 2])
@pytest.mark.parametrize("pinned", [False, True])
def test_group_host_operands_with_row_strides(backend, gpus, pinned):
    """Host matrices that are windows of wider arrays (lda > K, ldb > N, ldc, ldd > N): every copy is two-dimensional,
    B's bands over the GPUs' links included; K = 137 is odd so the last band is shorter; what lies outside the windows
    is not touched."""
    if backend.Device.count() < gpus:
        pytest.skip("needs two GPUs")
    lib = L.load()
    M, N, K = 1033, 260, 137
    lda, ldb, ldc, ldd = K + 5, N + 12, N + 4, N + 8
    rng = np.random.default_rng(17)
    held = []

    def host(rows, ld):
        x = rng.standard_normal(rows * ld).astype(np.float32)
        if not pinned:
            return x
        p = C.c_void_p()
        _check(lib.sb200_host_alloc(x.nbytes, C.byref(p)))
        held.append(p)
        v = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(x.size,))
        v[:] = x
        return v

    a, b, c, d = host(M, lda), host(K, ldb), host(M, ldc), host(M, ldd)
    d[:] = CANARY
    bias = rng.standard_normal(N).astype(np.float32)
    devs = [backend.Device.get(i).id for i in range(gpus)]
    grp = DeviceGroup(devs)
    try:
        _check(lib.sb200_gemm_sharded_host(grp.handle, L.MODE_3XTF32, M, N, K, a.ctypes.data, lda, b.ctypes.data, ldb, d.ctypes.data,
                                           ldd, 1.5, c.ctypes.data, ldc, 0.5, bias.ctypes.data, 1))
        dv = np.array(d).reshape(M, ldd)
        assert np.all(dv[:, N:] == CANARY)
        av = np.ascontiguousarray(np.array(a).reshape(M, lda)[:, :K]).ravel()
        bv = np.ascontiguousarray(np.array(b).reshape(K, ldb)[:, :N]).ravel()
        cv = np.ascontiguousarray(np.array(c).reshape(M, ldc)[:, :N]).ravel()
        ref = O.gemm(av, bv, M, N, K, 1.5, 0.5, cv, bias, 1)
        assert O.gemm_rel_error(dv[:, :N], ref) <= _tol(L.MODE_3XTF32, K)
    finally:
        grp.close()
        for p in held:
            _check(lib.sb200_host_free(p))
        backend.Device.set_current(backend.Device.get(0))
