"""Row-sharded GEMM with the gather fused into the epilogue, across two GPUs (one process per GPU).

Needs two B200s; skipped otherwise.  Each rank computes its row block and stores it into its own and the
peer's copy of D (peer memory mapped with sb200_ipc_open, plain stores over NVLink); after a host barrier both
copies must hold the whole product.  NVLS is switched off for the host-side process group, and no rank leaves
with work in flight.
"""
import ctypes as C
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, M, N, K, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from spoc_b200 import Backend, _lib as L
        from spoc_b200.plugin import _check
        from spoc_b200.sharding import row_block
        from tests import oracle_lib as O
        lib = L.load()
        backend = Backend()
        backend.Device.init()
        dev = backend.Device.get(rank)
        backend.Device.set_current(dev)
        a_full, b, c_full = O.fill(M * K, 61, 1), O.fill(K * N, 61, 2), O.fill(M * N, 61, 3)
        bias = O.fill(N, 61, 4, kind=1)
        r0, rows = row_block(M, world, rank)
        up = lambda arr: (lambda buf: (backend.Memory.host_to_device(src=arr, dst=buf), buf)[1])(backend.Memory.alloc(dev, arr.size, np.float32))
        A, B, Cm, Bi = up(np.ascontiguousarray(a_full[r0 * K:(r0 + rows) * K])), up(b), up(np.ascontiguousarray(c_full[r0 * N:(r0 + rows) * N])), up(bias)
        D = backend.Memory.alloc(dev, M * N, np.float32)
        backend.Memory.host_to_device(src=np.full(M * N, -7.0, np.float32), dst=D)
        handle = C.create_string_buffer(64)
        _check(lib.sb200_ipc_export(dev.id, D.ptr, handle))
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw)
        copies = [D.ptr]                                   # own copy first
        opened = []
        for r in range(world):
            if r != rank:
                p = C.c_uint64(0)
                _check(lib.sb200_ipc_open(dev.id, C.create_string_buffer(handles[r], 64), C.byref(p)))
                copies.append(p.value)
                opened.append(p.value)
        dist.barrier()                                      # every copy is initialised before anyone writes
        ptrs = (C.c_uint64 * world)(*copies)
        _check(lib.sb200_gemm_f32_gather(dev.id, 0, mode, rows, N, K, A.ptr, K, B.ptr, N, ptrs, world, r0, N, 1.5, Cm.ptr, N, 0.5,
                                         Bi.ptr, 1))
        backend.Device.synchronize(dev)
        dist.barrier()                                      # all ranks' stores have completed
        got = np.empty(M * N, np.float32)
        backend.Memory.device_to_host(src=D, dst=got)
        want = O.gemm(a_full, b, M, N, K, 1.5, 0.5, c_full, bias, 1)
        bound = (1e-5 * np.sqrt(K) if mode == L.MODE_3XTF32 else 2e-3) * 1.5 * np.sqrt(2)
        q.put((rank, O.gemm_rel_error(got.reshape(M, N), want) <= bound))
        dist.barrier()                                      # nobody unmaps while a peer may still read
        for p in opened:
            _check(lib.sb200_ipc_close(dev.id, p))
        for buf in (A, B, Cm, Bi, D):
            backend.Memory.free(buf)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", [3, 1])
def test_two_gpu_gather_fused_gemm(backend, mode):
    if backend.Device.count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, 1000, 520, 300, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results == {0: True, 1: True}
