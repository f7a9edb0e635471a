"""Row-block sharding of the GEMM / map path across the GPUs of one node.

Every output row depends on one row of A and all of B, and maps are
element-independent, so the path shards with no exchange step: rank r owns a
contiguous block of rows of A, C and D (or a contiguous index range of a map);
B and the bias are replicated.  The split rule for sizes that do not divide is
the reference's Vector.partition rule, `base + (i < rem)`
(sarek/core/Vector_storage.ml:261-272).  A gathered result is the
concatenation of the blocks, because row blocks of a row-major matrix are
contiguous.
"""
from __future__ import annotations

import importlib.util
import os


def partition(total: int, parts: int) -> list[tuple[int, int]]:
    """[(start, length)] for each part: the first `total % parts` parts get one extra element."""
    if parts <= 0 or total < 0:
        raise ValueError("partition needs parts > 0 and total >= 0")
    base, rem = divmod(total, parts)
    out, start = [], 0
    for i in range(parts):
        n = base + (1 if i < rem else 0)
        out.append((start, n))
        start += n
    return out


def row_block(m: int, world: int, rank: int) -> tuple[int, int]:
    """(first_row, rows) of rank `rank`."""
    return partition(m, world)[rank]


def gather_counts(m: int, n: int, world: int) -> list[int]:
    """Element counts of each rank's block of a row-major m x n result, in rank order."""
    return [rows * n for _, rows in partition(m, world)]


class DeviceGroup:
    """Several GPUs of this process driven through the library's group entry points (include/sb200.h:
    sb200_group_create, sb200_gemm_sharded, sb200_gemm_sharded_host).  The library owns the streams, the NCCL
    communicators and the replicas of B; this class only passes pointers and sizes, like the ctypes-foreign
    binding of an OCaml host would."""

    GATHER_NONE, GATHER_FUSED, GATHER_NCCL = 0, 1, 2

    def __init__(self, devices=None, ngpus: int | None = None):
        import ctypes as C
        from . import _lib as L
        from .plugin import _check
        self._C, self._L, self._check = C, L, _check
        self._lib = L.load()
        self._seen: dict = {}
        if devices is None:
            devices = list(range(ngpus if ngpus is not None else 1))
        self.devices = list(devices)
        if len(self.devices) > 1 and not os.environ.get("SAREK_B200_NCCL"):
            # a Python process usually also holds a framework with its own NCCL; point the library at that file so that
            # the process ends up with one NCCL whichever of the two is loaded first
            spec = importlib.util.find_spec("nvidia.nccl")
            for base in (list(spec.submodule_search_locations) if spec and spec.submodule_search_locations else []):
                cand = os.path.join(base, "lib", "libnccl.so.2")
                if os.path.exists(cand):
                    os.environ["SAREK_B200_NCCL"] = cand
                    break
        arr = (C.c_int * len(self.devices))(*self.devices)
        h = C.c_uint64(0)
        _check(self._lib.sb200_group_create(len(self.devices), arr, C.byref(h)))
        self.handle = h.value

    def __len__(self) -> int:
        return len(self.devices)

    def row_block(self, m: int, index: int) -> tuple[int, int]:
        C = self._C
        first, count = C.c_int64(0), C.c_int64(0)
        self._check(self._lib.sb200_row_block(m, len(self.devices), index, C.byref(first), C.byref(count)))
        return first.value, count.value

    def gemm(self, mode: int, m: int, n: int, k: int, a_shards, b: int, d, *, alpha=1.0, c_shards=None, beta=0.0, bias: int = 0,
             act: int = 0, gather: int = 0, b_resident: bool = False, lda=None, ldb=None, ldc=None, ldd=None) -> float:
        """Device-resident operands (device pointers as integers); returns the device time of the call in ms."""
        C, L = self._C, self._L
        g = len(self.devices)
        tab = lambda xs: (C.c_uint64 * g)(*[int(x or 0) for x in xs])
        flags = {0: 0, 1: L.SHARD_GATHER_FUSED, 2: L.SHARD_GATHER_NCCL}[gather] | (L.SHARD_B_RESIDENT if b_resident else 0)
        self._check(self._lib.sb200_gemm_sharded(self.handle, mode, m, n, k, tab(a_shards), k if lda is None else lda, int(b),
                                                 n if ldb is None else ldb, tab(d), n if ldd is None else ldd, alpha,
                                                 tab(c_shards) if c_shards is not None else None, n if ldc is None else ldc, beta,
                                                 int(bias), act, flags))
        ms = C.c_float(0)
        self._check(self._lib.sb200_group_last_ms(self.handle, C.byref(ms)))
        return ms.value

    PIN_MIN_BYTES = 16 << 20

    def _note_use(self, arr) -> None:
        """The policy of plugin.Vector for the arrays this group is handed: an array of 16 MiB or more that comes a second
        time is pinned in place (sb200_host_register) and held until close(), which unregisters it; later calls then move
        it by plain DMA instead of staging it through host threads.  SAREK_B200_PIN_VECTORS=0 switches this off."""
        if arr is None or arr.nbytes < self.PIN_MIN_BYTES or os.environ.get("SAREK_B200_PIN_VECTORS", "1") == "0":
            return
        key = arr.ctypes.data
        seen = self._seen.setdefault(key, [0, None])
        seen[0] += 1
        if seen[0] == 2 and seen[1] is None and self._lib.sb200_host_register(arr.ctypes.data_as(self._C.c_void_p), arr.nbytes) == 0:
            seen[1] = arr          # keeps the memory alive while it is registered

    def gemm_host(self, mode: int, m: int, n: int, k: int, a, b, d, *, alpha=1.0, c=None, beta=0.0, bias=None, act: int = 0) -> None:
        """Host operands (numpy float32 arrays, row-major contiguous); D is written in place."""
        for arr in (a, b, c, d):
            self._note_use(arr)
        ptr = lambda x: None if x is None else x.ctypes.data
        self._check(self._lib.sb200_gemm_sharded_host(self.handle, mode, m, n, k, ptr(a), k, ptr(b), n, ptr(d), n, alpha, ptr(c), n,
                                                      beta, ptr(bias), act))

    def close(self) -> None:
        for key, (_, arr) in list(self._seen.items()):
            if arr is not None:
                self._lib.sb200_host_unregister(arr.ctypes.data_as(self._C.c_void_p))
        self._seen.clear()
        if self.handle:
            self._check(self._lib.sb200_group_destroy(self.handle))
            self.handle = 0
