"""Small helpers for the GPU tests: device buffers through the plugin's Memory module."""
from __future__ import annotations

import ctypes as C

import numpy as np

from spoc_b200 import _lib as L
from spoc_b200.plugin import _check

CANARY = np.float32(-12345.678)


class Dev:
    """A float32 device buffer with `pad` canary elements on both sides of the payload."""

    def __init__(self, backend, device, n: int, pad: int = 64, offset: int = 0):
        self.backend, self.device = backend, device
        self.n, self.pad, self.offset = n, pad, offset
        self.total = n + 2 * pad + offset
        self.buf = backend.Memory.alloc(device, self.total, np.float32)
        self.clear()

    @property
    def ptr(self) -> int:
        return self.buf.ptr + 4 * (self.pad + self.offset)

    def clear(self):
        host = np.full(self.total, CANARY, dtype=np.float32)
        self.backend.Memory.host_to_device(src=host, dst=self.buf)

    def upload(self, arr: np.ndarray):
        arr = np.ascontiguousarray(arr, dtype=np.float32).ravel()
        assert arr.size == self.n
        host = np.full(self.total, CANARY, dtype=np.float32)
        host[self.pad + self.offset:self.pad + self.offset + self.n] = arr
        self.backend.Memory.host_to_device(src=host, dst=self.buf)
        return self

    def download(self, check_canary: bool = True) -> np.ndarray:
        host = np.empty(self.total, dtype=np.float32)
        self.backend.Memory.device_to_host(src=self.buf, dst=host)
        lo = self.pad + self.offset
        if check_canary:
            assert np.all(host[:lo] == CANARY), "write before the start of the buffer"
            assert np.all(host[lo + self.n:] == CANARY), "write past the end of the buffer"
        return host[lo:lo + self.n].copy()

    def free(self):
        self.backend.Memory.free(self.buf)


def dev_from(backend, device, arr, pad=64, offset=0) -> Dev:
    return Dev(backend, device, int(np.asarray(arr).size), pad, offset).upload(arr)


def gemm(backend, device, mode, M, N, K, A: Dev, B: Dev, D: Dev, alpha=1.0, C_: Dev | None = None, beta=0.0,
         bias: Dev | None = None, act=0, lda=None, ldb=None, ldd=None, ldc=None, stream=0):
    lib = L.load()
    _check(lib.sb200_gemm_f32(device.id, stream, mode, M, N, K, A.ptr, K if lda is None else lda, B.ptr,
                              N if ldb is None else ldb, D.ptr, N if ldd is None else ldd, alpha,
                              C_.ptr if C_ else 0, N if ldc is None else ldc, beta, bias.ptr if bias else 0, act))
    backend.Device.synchronize(device)
