"""sb200_kernel_launch_from_host: the launch that also brings over the vectors whose valid copy is still on the host
(Transfer.to_device of sarek/core/Execute.ml's run_vectors folded into the launch call).  Whatever route the uploads take
— row blocks pipelined with the GEMM when every host array is page-locked and the launch covers the whole product, whole
vectors first otherwise — the result is bit for bit that of uploading and then calling sb200_kernel_launch."""
import ctypes as C

import numpy as np
import pytest

from spoc_b200 import Vector, dims1d, dims2d, run_vectors, sarek_ir
from spoc_b200 import _lib as L
from spoc_b200.plugin import RSA_Buffer, RSA_Int32, _check
from tests import oracle_lib as O

pytestmark = pytest.mark.gpu

EPI = dict(alpha=1.5, beta=0.5, c="c", bias="bias", relu=True)


class _Pinned:
    """float32 host arrays in page-locked memory from the library's own allocator."""

    def __init__(self):
        self.ptrs = []

    def array(self, src: np.ndarray) -> np.ndarray:
        p = C.c_void_p()
        _check(L.load().sb200_host_alloc(max(src.nbytes, 4), C.byref(p)))
        self.ptrs.append(p)
        out = np.frombuffer((C.c_char * max(src.nbytes, 4)).from_address(p.value), dtype=np.float32)[:src.size]
        out[:] = src.ravel()
        return out

    def release(self):
        for p in self.ptrs:
            _check(L.load().sb200_host_free(p))
        self.ptrs = []


def _operands(M, N, K, seed):
    return (O.fill(M * K, seed, 1), O.fill(K * N, seed + 1, 1), O.fill(M * N, seed + 2, 1), O.fill(N, seed + 3, 1))


def _launch(backend, device, ir, shape, bufs, hosts, grid, block, copies=None):
    """bufs: device buffers of a, b, c, bias, d; hosts: same order, None where the device copy is current; copies: same
    order, the arrays results may be sent back to.  Returns the argument positions whose results are coming back."""
    M, N, K = shape
    args = []
    for buf, host, copy in zip(bufs, hosts, copies or [None] * len(bufs)):
        args += [RSA_Buffer(buf, buf.size, host, copy), RSA_Int32(buf.size)]
    args += [RSA_Int32(M), RSA_Int32(N), RSA_Int32(K)]
    return backend.run_source(source=ir, lang=backend.supported_source_langs[0], kernel_name="sarek_kern", block=block,
                              grid=grid, shared_mem=0, args=args)


def _download(backend, device, buf):
    out = np.empty(buf.size, dtype=np.float32)
    backend.Device.synchronize(device)
    backend.Memory.device_to_host(src=buf, dst=out)
    return out


@pytest.mark.parametrize("shape", [(1000, 520, 300), (2048, 1024, 512), (256 * 9 + 5, 136, 64), (3, 8, 5), (4096, 2048, 1024)])
@pytest.mark.parametrize("form", ["naive", "tiled"])
@pytest.mark.parametrize("memory", ["pinned", "pageable"])
def test_launch_from_host_equals_upload_then_launch(backend, device, shape, form, memory):
    M, N, K = shape
    a, b, c, bias = _operands(M, N, K, 11 * M + N)
    pin = _Pinned()
    try:
        host = [pin.array(x) if memory == "pinned" else x.copy() for x in (a, b, c, bias)]
        if form == "naive":
            ir, block, grid = sarek_ir.matmul_naive_ir(epilogue=EPI), dims1d(256), dims1d((M * N + 255) // 256)
        else:
            ir, block, grid = sarek_ir.matmul_tiled_ir(epilogue=EPI), dims2d(16, 16), dims2d((N + 15) // 16, (M + 15) // 16)
        sizes = (M * K, K * N, M * N, N, M * N)
        ref_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
        new_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
        try:
            for buf, x in zip(ref_bufs[:4], (a, b, c, bias)):
                backend.Memory.host_to_device(src=x, dst=buf)
            _launch(backend, device, ir, shape, ref_bufs, [None] * 5, grid, block)
            want = _download(backend, device, ref_bufs[4])
            _launch(backend, device, ir, shape, new_bufs, host + [None], grid, block)
            for h in host:          # the call has returned: the host arrays are the caller's again
                h[:] = -3.0
            got = _download(backend, device, new_bufs[4])
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            # the uploaded operands are on the device as whole vectors, as after Transfer.to_device
            assert np.array_equal(_download(backend, device, new_bufs[0]), a)
            assert np.array_equal(_download(backend, device, new_bufs[2]), c)
        finally:
            for buf in ref_bufs + new_bufs:
                backend.Memory.free(buf)
    finally:
        pin.release()


def test_only_some_operands_from_the_host(backend, device):
    """B already resident (the usual case of a weight matrix), A and C still on the host."""
    M, N, K = 2048, 768, 640
    a, b, c, bias = _operands(M, N, K, 5)
    pin = _Pinned()
    ir, block, grid = sarek_ir.matmul_naive_ir(epilogue=EPI), dims1d(256), dims1d((M * N + 255) // 256)
    sizes = (M * K, K * N, M * N, N, M * N)
    ref_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
    new_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
    try:
        for buf, x in zip(ref_bufs[:4], (a, b, c, bias)):
            backend.Memory.host_to_device(src=x, dst=buf)
        backend.Memory.host_to_device(src=b, dst=new_bufs[1])
        backend.Memory.host_to_device(src=bias, dst=new_bufs[3])
        _launch(backend, device, ir, (M, N, K), ref_bufs, [None] * 5, grid, block)
        _launch(backend, device, ir, (M, N, K), new_bufs, [pin.array(a), None, pin.array(c), None, None], grid, block)
        assert np.array_equal(_download(backend, device, new_bufs[4]), _download(backend, device, ref_bufs[4]))
    finally:
        for buf in ref_bufs + new_bufs:
            backend.Memory.free(buf)
        pin.release()


def test_partial_launch_from_the_host_computes_the_same_elements(backend, device):
    """A launch that covers only part of the product is not pipelined; the elements it covers come out the same and the
    rest of the result buffer is left alone."""
    M, N, K = 600, 200, 96
    a, b, c, bias = _operands(M, N, K, 9)
    pin = _Pinned()
    ir, block = sarek_ir.matmul_naive_ir(epilogue=EPI), dims1d(256)
    grid = dims1d((M * N // 2) // 256)
    sizes = (M * K, K * N, M * N, N, M * N)
    ref_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
    new_bufs = [backend.Memory.alloc(device, n, np.float32) for n in sizes]
    try:
        marker = np.full(M * N, 777.0, dtype=np.float32)
        for bufs in (ref_bufs, new_bufs):
            backend.Memory.host_to_device(src=marker, dst=bufs[4])
        for buf, x in zip(ref_bufs[:4], (a, b, c, bias)):
            backend.Memory.host_to_device(src=x, dst=buf)
        _launch(backend, device, ir, (M, N, K), ref_bufs, [None] * 5, grid, block)
        _launch(backend, device, ir, (M, N, K), new_bufs, [pin.array(x) for x in (a, b, c, bias)] + [None], grid, block)
        want, got = _download(backend, device, ref_bufs[4]), _download(backend, device, new_bufs[4])
        assert np.array_equal(got, want)
        assert np.all(got[grid.x * 256:] == 777.0) and not np.all(got[:grid.x * 256] == 777.0)
    finally:
        for buf in ref_bufs + new_bufs:
            backend.Memory.free(buf)
        pin.release()


def test_map_kernel_from_the_host(backend, device):
    n = 100003
    a, b = O.fill(n, 1, 1), O.fill(n, 2, 1)
    va, vb, vc = Vector(backend, a.copy()), Vector(backend, b.copy()), Vector(backend, np.zeros(n, dtype=np.float32))
    try:
        run_vectors(backend, device=device, ir=sarek_ir.vector_add_ir(), args=[va, vb, vc, ("int32", n)],
                    block=dims1d(256), grid=dims1d((n + 255) // 256))
        assert va.location == Vector.STALE_CPU and vc.location == Vector.STALE_CPU
        assert np.array_equal(vc.to_array(), a + b)       # one float32 rounding of the exact sum either way
    finally:
        for v in (va, vb, vc):
            v.free()


def test_run_vectors_repeated_with_large_vectors(backend, device):
    """Vectors of 16 MiB: first launch from pageable arrays, later ones from arrays the plugin has pinned in place (the
    pipelined route); every launch gives the same bits, and new host contents are picked up."""
    M = N = K = 2048
    a, b, c, bias = _operands(M, N, K, 21)
    ir = sarek_ir.matmul_naive_ir(epilogue=EPI)
    vecs = [Vector(backend, x.copy()) for x in (a, b, c, bias)] + [Vector(backend, np.zeros(M * N, dtype=np.float32))]
    try:
        results = []
        for _ in range(3):
            for v in vecs[:4]:
                v.location = Vector.CPU
            run_vectors(backend, device=device, ir=ir, args=vecs + [("int32", M), ("int32", N), ("int32", K)],
                        block=dims1d(256), grid=dims1d((M * N + 255) // 256))
            results.append(vecs[4].to_array().copy())
        assert vecs[0]._pinned and vecs[1]._pinned and not vecs[3]._pinned
        assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])
        rows = np.arange(0, M, 97)
        ref = np.maximum(1.5 * (a.reshape(M, K)[rows].astype(np.float64) @ b.reshape(K, N).astype(np.float64))
                         + 0.5 * c.reshape(M, N)[rows] + bias, 0.0)
        err = np.abs(results[0].reshape(M, N)[rows] - ref).max() / np.sqrt(np.mean(ref * ref))
        assert err < 1e-5 * np.sqrt(K)
        vecs[0].host[:] = 0.0                      # A = 0: the product term vanishes
        vecs[0].location = Vector.CPU
        run_vectors(backend, device=device, ir=ir, args=vecs + [("int32", M), ("int32", N), ("int32", K)],
                    block=dims1d(256), grid=dims1d((M * N + 255) // 256))
        want = np.maximum(np.float32(0.5) * c.reshape(M, N) + bias, np.float32(0.0))
        assert np.allclose(vecs[4].to_array().reshape(M, N), want, rtol=1e-6, atol=1e-6)
    finally:
        for v in vecs:
            v.free()


@pytest.mark.parametrize("shape,whole", [((1024, 512, 256), True), ((2304, 256, 128), True), ((700, 300, 64), False)])
@pytest.mark.parametrize("from_host", ["all", "operands", "none"])
def test_longer_vectors_and_the_result_sent_back_behind_the_kernel(backend, device, shape, whole, from_host):
    """Vectors longer than the product needs arrive whole (tails and the old contents of D's vector included), and the
    result is on the host after sb200_prefetch_wait without a download call — on the pipelined route (whole launch,
    operands from the host), behind a plain launch (operands resident) and behind a partial launch."""
    M, N, K = shape
    extra = 1000
    a, b, c, bias = (np.concatenate([x, O.fill(extra, 40 + i, 1)]) for i, x in enumerate(_operands(M, N, K, 3)))
    d0 = O.fill(M * N + extra, 50, 1)
    pin = _Pinned()
    ir, block = sarek_ir.matmul_naive_ir(epilogue=EPI), dims1d(256)
    covered = M * N if whole else (M * N // 2) // 256 * 256
    grid = dims1d((covered + 255) // 256)
    ref_bufs = [backend.Memory.alloc(device, x.size, np.float32) for x in (a, b, c, bias, d0)]
    new_bufs = [backend.Memory.alloc(device, x.size, np.float32) for x in (a, b, c, bias, d0)]
    try:
        for buf, x in zip(ref_bufs, (a, b, c, bias, d0)):
            backend.Memory.host_to_device(src=x, dst=buf)
        _launch(backend, device, ir, shape, ref_bufs, [None] * 5, grid, block)
        want = _download(backend, device, ref_bufs[4])
        assert np.array_equal(want[covered:], d0[covered:])
        host = [pin.array(x) for x in (a, b, c, bias, d0)]
        resident = {"all": [], "operands": [4], "none": [0, 1, 2, 3, 4]}[from_host]
        for i in resident:
            backend.Memory.host_to_device(src=(a, b, c, bias, d0)[i], dst=new_bufs[i])
        if 4 in resident:
            host[4][:] = -1.0          # the host copy of D is stale everywhere, beyond the product too
        coming = _launch(backend, device, ir, shape, new_bufs, [None if i in resident else host[i] for i in range(5)], grid, block,
                         copies=[None, None, None, None, host[4]])
        assert coming == {8}                       # the fifth vector's buffer argument
        _check(L.load().sb200_prefetch_wait(device.id))
        assert np.array_equal(host[4].view(np.uint32), want.view(np.uint32))
        for buf, x in zip(new_bufs[:4], (a, b, c, bias)):
            assert np.array_equal(_download(backend, device, buf), x)
        assert np.array_equal(_download(backend, device, new_bufs[4]), want)
    finally:
        for buf in ref_bufs + new_bufs:
            backend.Memory.free(buf)
        pin.release()


def test_pageable_result_array_is_not_prefetched(backend, device):
    M, N, K = 256, 128, 64
    a, b, c, bias = _operands(M, N, K, 8)
    ir, block, grid = sarek_ir.matmul_naive_ir(epilogue=EPI), dims1d(256), dims1d((M * N + 255) // 256)
    bufs = [backend.Memory.alloc(device, n, np.float32) for n in (M * K, K * N, M * N, N, M * N)]
    try:
        d_host = np.full(M * N, 5.0, dtype=np.float32)
        coming = _launch(backend, device, ir, (M, N, K), bufs, [a, b, c, bias, None], grid, block,
                         copies=[None, None, None, None, d_host])
        assert coming == set()
        _check(L.load().sb200_prefetch_wait(device.id))
        assert np.all(d_host == 5.0)
        want = O.gemm(a, b, M, N, K, alpha=1.5, beta=0.5, cin=c, bias=bias, act=L.ACT_RELU)
        assert O.gemm_rel_error(_download(backend, device, bufs[4]).reshape(M, N), want) < 1e-5 * np.sqrt(K)
    finally:
        for buf in bufs:
            backend.Memory.free(buf)


def test_null_table_and_short_vectors_are_refused(backend, device):
    lib = L.load()
    ir = sarek_ir.matmul_naive_ir()
    k = backend.Kernel.compile_cached(device, name="sarek_kern", source=ir)
    g, b = (C.c_uint32 * 3)(1, 1, 1), (C.c_uint32 * 3)(256, 1, 1)
    arr = (L.Arg * 1)()
    assert lib.sb200_kernel_launch_from_host(k.handle, arr, 1, None, None, None, g, b, 0, 0) == L.ERR_INVALID_VALUE
    hp, pre = (C.c_void_p * 1)(), (C.c_int32 * 1)()
    assert lib.sb200_kernel_launch_from_host(k.handle, arr, 1, hp, None, pre, g, b, 0, 0) == L.ERR_INVALID_VALUE


# ---- element-wise operators by chunks -----------------------------------------------------------------------------
N_MAP = (8 << 20) + 12345          # 32 MiB per vector and a ragged end


def _map_launch(backend, device, ir, bufs, hosts, copies, scalars, n):
    args = []
    for buf, host, copy in zip(bufs, hosts, copies):
        args += [RSA_Buffer(buf, buf.size, host, copy), RSA_Int32(buf.size)]
    args += scalars
    return backend.run_source(source=ir, lang=backend.supported_source_langs[0], kernel_name="sarek_kern", block=dims1d(256),
                              grid=dims1d((n + 255) // 256), shared_mem=0, args=args)


@pytest.mark.parametrize("kernel", ["vector_add", "stream_triad", "chain"])
@pytest.mark.parametrize("extra", [0, 777])
def test_map_from_pinned_host_arrays_by_chunks(backend, device, kernel, extra):
    """Large vectors from page-locked arrays: uploaded, computed and sent back chunk by chunk; the same bits as upload,
    one launch, download; vectors longer than the launch covers arrive whole and come back whole."""
    from spoc_b200.plugin import RSA_Float32
    n, length = N_MAP, N_MAP + extra
    x, y, z0 = O.fill(length, 31, 1), O.fill(length, 31, 2), O.fill(length, 31, 3)
    if kernel == "vector_add":       # a, b -> c
        ir, order, out, scalars = sarek_ir.vector_add_ir(), (x, y, z0), 2, [RSA_Int32(n)]
    elif kernel == "stream_triad":   # a <- b + c * s
        ir, order, out, scalars = sarek_ir.stream_triad_ir(), (z0, x, y), 0, [RSA_Float32(3.0), RSA_Int32(n)]
    else:                            # d <- (b + 3c)^2 + b, unguarded: the launch covers whole blocks of 256
        n = N_MAP // 256 * 256
        ir, order, out, scalars = sarek_ir.chain_fused_ir(3.0), (z0, x, y), 0, []
    pin = _Pinned()
    ref_bufs = [backend.Memory.alloc(device, length, np.float32) for _ in range(3)]
    new_bufs = [backend.Memory.alloc(device, length, np.float32) for _ in range(3)]
    try:
        for buf, v in zip(ref_bufs, order):
            backend.Memory.host_to_device(src=v, dst=buf)
        assert _map_launch(backend, device, ir, ref_bufs, [None] * 3, [None] * 3, scalars, n) == set()
        want = _download(backend, device, ref_bufs[out])
        assert np.array_equal(want[n:], order[out][n:])             # beyond the launch: untouched
        host = [pin.array(v) for v in order]
        coming = _map_launch(backend, device, ir, new_bufs, host, [host[i] if i == out else None for i in range(3)], scalars, n)
        assert coming == {2 * out}
        _check(L.load().sb200_prefetch_wait(device.id))
        assert np.array_equal(host[out].view(np.uint32), want.view(np.uint32))
        for i in range(3):
            assert np.array_equal(_download(backend, device, new_bufs[i]), want if i == out else order[i])
    finally:
        for buf in ref_bufs + new_bufs:
            backend.Memory.free(buf)
        pin.release()


def test_map_in_place_from_the_host(backend, device):
    """stream_triad with its output bound to the buffer of its first input: a <- a + c * s."""
    from spoc_b200.plugin import RSA_Float32
    n = N_MAP
    a, c = O.fill(n, 32, 1), O.fill(n, 32, 2)
    pin = _Pinned()
    A, Cb = backend.Memory.alloc(device, n, np.float32), backend.Memory.alloc(device, n, np.float32)
    try:
        ha, hc = pin.array(a), pin.array(c)
        coming = _map_launch(backend, device, sarek_ir.stream_triad_ir(), [A, A, Cb], [ha, ha, hc], [ha, None, None],
                             [RSA_Float32(0.5), RSA_Int32(n)], n)
        assert coming == {0}
        _check(L.load().sb200_prefetch_wait(device.id))
        want = (a.astype(np.float64) + c.astype(np.float64) * 0.5).astype(np.float32)
        assert np.array_equal(np.array(ha), want)
        assert np.array_equal(_download(backend, device, A), want)
    finally:
        backend.Memory.free(A)
        backend.Memory.free(Cb)
        pin.release()


def test_run_vectors_on_large_map_vectors(backend, device):
    """Through Vector / run_vectors: pageable on the first launch, pinned in place later, chunked from then on."""
    n = N_MAP
    b, c = O.fill(n, 33, 1), O.fill(n, 33, 2)
    vb, vc, vd = Vector(backend, b.copy()), Vector(backend, c.copy()), Vector(backend, np.zeros(n, dtype=np.float32))
    want = (b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)
    try:
        for rep in range(4):
            vb.location = vc.location = Vector.CPU
            run_vectors(backend, device=device, ir=sarek_ir.vector_add_ir(), args=[vb, vc, vd, ("int32", n)], block=dims1d(256),
                        grid=dims1d((n + 255) // 256))
            got = vd.to_array()
            assert np.array_equal(got, want), rep
            vd.host[:] = -1.0
            vd.location = Vector.STALE_CPU if rep % 2 else Vector.BOTH   # sometimes the host copy is declared current
            if vd.location == Vector.BOTH:
                vd.host[:] = want
        assert vb._pinned and vd._pinned
    finally:
        for v in (vb, vc, vd):
            v.free()
