"""Host-side mirror of the plugin interface, over the C ABI.

The reference's host language is OCaml and no OCaml toolchain exists where
this repository is built, so the part of the plugin that sits above the C ABI
is written here with the names, argument meaning and error behaviour of the
reference interface it stands for:

* ``Backend`` has the members of ``Framework_sig.BACKEND``
  (spoc/framework/Framework_sig.ml:137-350) in the arrangement of
  sarek-cuda/Cuda_plugin.ml:146-224: ``Device``, ``Stream``, ``Memory``,
  ``Event``, ``Kernel``, ``generate_source``, ``run_source``,
  ``execution_model = "JIT"``, ``supported_source_langs``.
* ``Vector`` and ``run_vectors`` follow ``Spoc_core.Vector`` /
  ``Sarek.Execute.run_vectors`` (sarek/core/Vector.ml, sarek/sarek/Execute.ml:
  197-216,231-304,520-543): lazy device allocation, host->device transfer on
  first use, a vector expands to (buffer, int32 length), every vector argument
  is stale on the CPU after a launch (Execute.ml:321-335).

Errors surface as exceptions, like ``Cuda_api.Cuda_error`` (Cuda_api.ml:27-31)
and ``Backend_error`` (spoc/framework/Backend_error.ml:21-78).  Nothing here
computes: every operation is a call into libsarek_b200.so.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from . import _lib as L


class BackendError(RuntimeError):
    """Carries the library's status code and message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[sarek-b200] error {code}: {message}")
        self.code = code
        self.message = message


class UnsupportedConstruct(BackendError):
    """The IR is not a kernel this backend runs (Backend_error.Unsupported_construct)."""


def _check(code: int) -> None:
    if code == 0:
        return
    msg = L.load().sb200_last_error_string().decode("utf-8", "replace")
    if code == L.ERR_UNSUPPORTED:
        raise UnsupportedConstruct(code, msg)
    raise BackendError(code, msg)


@dataclass(frozen=True)
class Dims:
    """Framework_sig.dims (spoc/framework/Framework_sig.ml:17)."""
    x: int = 1
    y: int = 1
    z: int = 1


def dims1d(x: int) -> Dims:
    return Dims(x, 1, 1)


def dims2d(x: int, y: int) -> Dims:
    return Dims(x, y, 1)


# ---------------------------------------------------------------- Device
class _Device:
    @dataclass(frozen=True)
    class T:
        id: int
        name: str
        total_mem: int
        compute_capability: tuple[int, int]
        sm_count: int
        max_shared_per_block: int
        l2_bytes: int

    def __init__(self) -> None:
        self._current = 0
        self._cache: dict[int, "_Device.T"] = {}   # device properties are slow to query: ask once

    def init(self) -> None:
        _check(L.load().sb200_init())

    def count(self) -> int:
        n = C.c_int(0)
        _check(L.load().sb200_device_count(C.byref(n)))
        return n.value

    def get(self, idx: int) -> "_Device.T":
        d = self._cache.get(idx)
        if d is None:
            info = L.DeviceInfo()
            _check(L.load().sb200_device_get_info(idx, C.byref(info)))
            d = self._cache[idx] = _Device.T(idx, info.name.decode(), info.total_mem, (info.cc_major, info.cc_minor),
                                             info.sm_count, info.max_shared_per_block, info.l2_bytes)
        return d

    def id(self, d: "_Device.T") -> int:
        return d.id

    def name(self, d: "_Device.T") -> str:
        return d.name

    def capabilities(self, d: "_Device.T") -> dict:
        return {"compute_capability": d.compute_capability, "multiprocessor_count": d.sm_count,
                "max_shared_memory": d.max_shared_per_block, "total_global_mem": d.total_mem,
                "supports_fp64": True, "supports_atomics": True, "warp_size": 32, "is_cpu": False}

    def set_current(self, d: "_Device.T") -> None:
        _check(L.load().sb200_device_set_current(d.id))
        self._current = d.id

    def get_current_device(self) -> int:
        return self._current

    def synchronize(self, d: "_Device.T") -> None:
        _check(L.load().sb200_device_synchronize(d.id))


# ---------------------------------------------------------------- Stream
class _Stream:
    @dataclass
    class T:
        dev: int
        handle: int

    def create(self, d: _Device.T) -> "_Stream.T":
        h = C.c_uint64(0)
        _check(L.load().sb200_stream_create(d.id, C.byref(h)))
        return _Stream.T(d.id, h.value)

    def wrap(self, d: _Device.T, native: int) -> "_Stream.T":
        h = C.c_uint64(0)
        _check(L.load().sb200_stream_wrap(d.id, native, C.byref(h)))
        return _Stream.T(d.id, h.value)

    def destroy(self, s: "_Stream.T") -> None:
        _check(L.load().sb200_stream_destroy(s.dev, s.handle))
        s.handle = 0

    def synchronize(self, s: "_Stream.T") -> None:
        _check(L.load().sb200_stream_synchronize(s.dev, s.handle))

    def default(self, d: _Device.T) -> "_Stream.T":
        return _Stream.T(d.id, 0)


# ---------------------------------------------------------------- Memory
class _Memory:
    @dataclass
    class Buffer:
        dev: int
        ptr: int
        size: int       # elements
        elem_size: int  # bytes

    def alloc(self, d: _Device.T, size: int, dtype=np.float32) -> "_Memory.Buffer":
        return self.alloc_custom(d, size=size, elem_size=np.dtype(dtype).itemsize)

    def alloc_custom(self, d: _Device.T, *, size: int, elem_size: int) -> "_Memory.Buffer":
        p = C.c_uint64(0)
        _check(L.load().sb200_mem_alloc(d.id, size * elem_size, C.byref(p)))
        return _Memory.Buffer(d.id, p.value, size, elem_size)

    def alloc_zero_copy(self, d: _Device.T, host: np.ndarray):
        return None  # discrete GPU: no zero-copy, as in Cuda_plugin_base

    def free(self, b: "_Memory.Buffer") -> None:
        _check(L.load().sb200_mem_free(b.dev, b.ptr))  # idempotent in the library

    def host_to_device(self, *, src: np.ndarray, dst: "_Memory.Buffer") -> None:
        src = np.ascontiguousarray(src)
        nbytes = min(src.nbytes, dst.size * dst.elem_size)
        _check(L.load().sb200_memcpy_htod(dst.dev, dst.ptr, src.ctypes.data_as(C.c_void_p), nbytes))

    def device_to_host(self, *, src: "_Memory.Buffer", dst: np.ndarray) -> None:
        assert dst.flags["C_CONTIGUOUS"]
        nbytes = min(dst.nbytes, src.size * src.elem_size)
        _check(L.load().sb200_memcpy_dtoh(src.dev, dst.ctypes.data_as(C.c_void_p), src.ptr, nbytes))

    def host_ptr_to_device(self, *, src_ptr: int, byte_size: int, dst: "_Memory.Buffer") -> None:
        _check(L.load().sb200_memcpy_htod(dst.dev, dst.ptr, C.c_void_p(src_ptr), byte_size))

    def device_to_host_ptr(self, *, src: "_Memory.Buffer", dst_ptr: int, byte_size: int) -> None:
        _check(L.load().sb200_memcpy_dtoh(src.dev, C.c_void_p(dst_ptr), src.ptr, byte_size))

    def device_to_device(self, *, src: "_Memory.Buffer", dst: "_Memory.Buffer") -> None:
        _check(L.load().sb200_memcpy_dtod(dst.dev, dst.ptr, src.ptr, min(src.size * src.elem_size, dst.size * dst.elem_size)))

    def size(self, b: "_Memory.Buffer") -> int:
        return b.size

    def device_ptr(self, b: "_Memory.Buffer") -> int:
        return b.ptr

    def is_zero_copy(self, b: "_Memory.Buffer") -> bool:
        return False


# ----------------------------------------------------------------- Event
class _Event:
    @dataclass
    class T:
        dev: int
        handle: int

    def __init__(self, device: _Device) -> None:
        self._device = device

    def create(self) -> "_Event.T":
        h = C.c_uint64(0)
        dev = self._device.get_current_device()
        _check(L.load().sb200_event_create(dev, C.byref(h)))
        return _Event.T(dev, h.value)

    def destroy(self, e: "_Event.T") -> None:
        _check(L.load().sb200_event_destroy(e.dev, e.handle))
        e.handle = 0

    def record(self, e: "_Event.T", s: _Stream.T) -> None:
        _check(L.load().sb200_event_record(e.dev, e.handle, s.handle))

    def synchronize(self, e: "_Event.T") -> None:
        _check(L.load().sb200_event_synchronize(e.dev, e.handle))

    def elapsed(self, *, start: "_Event.T", stop: "_Event.T") -> float:
        ms = C.c_float(0)
        _check(L.load().sb200_event_elapsed_ms(start.dev, start.handle, stop.handle, C.byref(ms)))
        return ms.value


# ---------------------------------------------------------------- Kernel
class _Kernel:
    @dataclass
    class T:
        dev: int
        handle: int
        name: str

        @property
        def kind(self) -> int:
            k = C.c_int(0)
            _check(L.load().sb200_kernel_kind(self.handle, C.byref(k)))
            return k.value

        def describe(self) -> str:
            buf = C.create_string_buffer(512)
            _check(L.load().sb200_kernel_describe(self.handle, buf, 512))
            return buf.value.decode()

    class Args:
        """Positional argument list; like the reference's, set_arg_* ignore their
        index and append in call order (sarek-cuda/Cuda_plugin_base.ml:268-281)."""

        def __init__(self) -> None:
            self.items: list[L.Arg] = []

    def __init__(self) -> None:
        self._cache: dict[tuple[int, str], "_Kernel.T"] = {}

    def compile(self, d: _Device.T, *, name: str, source: str) -> "_Kernel.T":
        h = C.c_uint64(0)
        _check(L.load().sb200_kernel_compile(d.id, source.encode(), name.encode(), C.byref(h)))
        return _Kernel.T(d.id, h.value, name)

    def compile_cached(self, d: _Device.T, *, name: str, source: str) -> "_Kernel.T":
        key = (d.id, source)
        k = self._cache.get(key)
        if k is None:
            k = self._cache[key] = self.compile(d, name=name, source=source)
        return k

    def clear_cache(self) -> None:
        for k in self._cache.values():
            L.load().sb200_kernel_destroy(k.handle)
        self._cache.clear()

    def create_args(self) -> "_Kernel.Args":
        return _Kernel.Args()

    @staticmethod
    def _push(args: "_Kernel.Args", tag: int, field: str, value) -> None:
        a = L.Arg()
        a.tag = tag
        setattr(a.v, field, value)
        args.items.append(a)

    def set_arg_buffer(self, args, _idx: int, buf: _Memory.Buffer) -> None:
        self._push(args, L.ARG_BUFFER, "buffer", buf.ptr)

    def set_arg_ptr(self, args, _idx: int, ptr: int) -> None:
        self._push(args, L.ARG_BUFFER, "buffer", ptr)

    def set_arg_int32(self, args, _idx: int, v: int) -> None:
        self._push(args, L.ARG_I32, "i32", int(v))

    def set_arg_int64(self, args, _idx: int, v: int) -> None:
        self._push(args, L.ARG_I64, "i64", int(v))

    def set_arg_float32(self, args, _idx: int, v: float) -> None:
        self._push(args, L.ARG_F32, "f32", float(v))

    def set_arg_float64(self, args, _idx: int, v: float) -> None:
        self._push(args, L.ARG_F64, "f64", float(v))

    def launch(self, k: "_Kernel.T", *, args: "_Kernel.Args", grid: Dims, block: Dims, shared_mem: int = 0,
               stream: _Stream.T | None = None, host_arrays: dict | None = None, host_copies: dict | None = None) -> set:
        """host_arrays maps argument positions (of buffer arguments) to host arrays the buffers are to be filled from
        first: the launch then goes through sb200_kernel_launch_from_host, which uploads and launches in one call and
        overlaps the two where it can.  host_copies maps positions to the arrays that hold the vectors' host copies;
        the positions whose result the library is already sending back there are returned (complete after
        sb200_prefetch_wait)."""
        n = len(args.items)
        arr = (L.Arg * max(n, 1))(*args.items)
        g = (C.c_uint32 * 3)(grid.x, grid.y, grid.z)
        b = (C.c_uint32 * 3)(block.x, block.y, block.z)
        if host_arrays or host_copies:
            host_arrays, host_copies = host_arrays or {}, host_copies or {}
            hp = (C.c_void_p * max(n, 1))(*[host_arrays[i].ctypes.data if i in host_arrays else None for i in range(n)])
            ho = (C.c_void_p * max(n, 1))(*[host_copies[i].ctypes.data if i in host_copies else None for i in range(n)])
            pre = (C.c_int32 * max(n, 1))()
            _check(L.load().sb200_kernel_launch_from_host(k.handle, arr, n, hp, ho, pre, g, b, shared_mem,
                                                          stream.handle if stream else 0))
            return {i for i in range(n) if pre[i]}
        _check(L.load().sb200_kernel_launch(k.handle, arr, n, g, b, shared_mem, stream.handle if stream else 0))
        return set()


# ------------------------------------------------------- run_source args
@dataclass
class RSA_Buffer:
    buffer: _Memory.Buffer
    length: int
    host: np.ndarray | None = None   # set when the device buffer has yet to be filled from this host array
    host_copy: np.ndarray | None = None   # the page-locked array a result may be sent back to behind the kernel


@dataclass
class RSA_Int32:
    value: int


@dataclass
class RSA_Int64:
    value: int


@dataclass
class RSA_Float32:
    value: float


@dataclass
class RSA_Float64:
    value: float


class Backend:
    """The ``(module BACKEND)`` value registered under ``name``."""

    name = "B200"
    version = (1, 0, 0)
    execution_model = "JIT"
    supported_source_langs = ["SarekIR_sexp"]

    def __init__(self) -> None:
        self.Device = _Device()
        self.Stream = _Stream()
        self.Memory = _Memory()
        self.Event = _Event(self.Device)
        self.Kernel = _Kernel()

    def is_available(self) -> bool:
        try:
            return self.Device.count() > 0
        except (L.LibraryMissing, OSError, BackendError):
            return False

    def generate_source(self, ir: str, block: Dims | None = None) -> str | None:
        """IR -> source text.  The IR already is its own source language here."""
        return ir

    def enable_profiling(self) -> None:
        _check(L.load().sb200_enable_profiling(1))

    def disable_profiling(self) -> None:
        _check(L.load().sb200_enable_profiling(0))

    def profile_gemm_read(self, d: _Device.T) -> dict:
        n, a, b = C.c_uint64(0), C.c_double(0), C.c_double(0)
        _check(L.load().sb200_profile_gemm_read(d.id, C.byref(n), C.byref(a), C.byref(b)))
        return {"calls": n.value, "prep_ms": a.value, "main_ms": b.value}

    def execute_direct(self, *a, **k):
        raise BackendError(L.ERR_UNSUPPORTED, "execute_direct: B200 is a JIT-model backend")

    def run_source(self, *, source: str, lang: str, kernel_name: str, block: Dims, grid: Dims, shared_mem: int,
                   args: Sequence, stream: _Stream.T | None = None) -> set:
        """sarek-cuda/Cuda_plugin.ml:174-210: compile (cached), bind arguments in order, launch.  Returns the positions
        of the buffer arguments whose results are on their way back to their host_copy arrays."""
        if lang not in self.supported_source_langs:
            raise BackendError(L.ERR_UNSUPPORTED, f"run_source: source language {lang!r} not supported")
        dev = self.Device.get(self.Device.get_current_device())
        k = self.Kernel.compile_cached(dev, name=kernel_name, source=source)
        ka = self.Kernel.create_args()
        host_arrays, host_copies = {}, {}
        for i, a in enumerate(args):
            if isinstance(a, RSA_Buffer):
                self.Kernel.set_arg_buffer(ka, i, a.buffer)
                if a.host is not None:
                    host_arrays[i] = a.host
                if a.host_copy is not None:
                    host_copies[i] = a.host_copy
            elif isinstance(a, RSA_Int32):
                self.Kernel.set_arg_int32(ka, i, a.value)
            elif isinstance(a, RSA_Int64):
                self.Kernel.set_arg_int64(ka, i, a.value)
            elif isinstance(a, RSA_Float32):
                self.Kernel.set_arg_float32(ka, i, a.value)
            elif isinstance(a, RSA_Float64):
                self.Kernel.set_arg_float64(ka, i, a.value)
            else:
                raise BackendError(L.ERR_ARGS, f"run_source: unsupported argument {a!r}")
        return self.Kernel.launch(k, args=ka, grid=grid, block=block, shared_mem=shared_mem, stream=stream,
                                  host_arrays=host_arrays, host_copies=host_copies)

    # -- the direct operators and settings (extras beyond BACKEND) ----------
    def set_mode(self, mode: int) -> None:
        _check(L.load().sb200_set_mode(mode))

    def get_mode(self) -> int:
        m = C.c_int(0)
        _check(L.load().sb200_get_mode(C.byref(m)))
        return m.value

    def set_gemm_variant(self, variant: int) -> None:
        """0 automatic, 1 single-CTA tiles, 2 CTA pairs."""
        _check(L.load().sb200_set_gemm_variant(variant))

    def launch_count(self) -> int:
        n = C.c_uint64(0)
        _check(L.load().sb200_launch_count(C.byref(n)))
        return n.value


# --------------------------------------------------- Vector / run_vectors
class Vector:
    """Spoc_core.Vector for float32: a host array plus a lazily created device
    buffer and a location state (sarek/core/Vector_types.ml:198-229)."""

    CPU, BOTH, STALE_CPU = "CPU", "Both", "Stale_CPU"

    PIN_MIN_BYTES = 16 << 20   # vectors at least this large are pinned in place on their second transfer

    def __init__(self, backend: Backend, host: np.ndarray):
        assert host.dtype == np.float32 and host.ndim == 1 and host.flags["C_CONTIGUOUS"]
        self.backend = backend
        self.host = host
        self.buffer: _Memory.Buffer | None = None
        self.location = Vector.CPU
        self._transfers = 0
        self._pinned = False
        self._prefetch_dev = None    # device whose outbound stream is bringing the result back to self.host

    def _note_transfer(self) -> None:
        """A vector owns its host array for its whole life (as Spoc_core.Vector owns its Bigarray), so the array can be
        pinned in place: the first large transfer goes through the staged pageable copier, and a vector that is moved a
        second time is registered with the driver (sb200_host_register) so that this and every later transfer run at the
        pinned rate.  SAREK_B200_PIN_VECTORS=0 switches this off; free() unregisters."""
        self._transfers += 1
        if (self._transfers == 2 and not self._pinned and self.host.nbytes >= Vector.PIN_MIN_BYTES
                and os.environ.get("SAREK_B200_PIN_VECTORS", "1") != "0"):
            if L.load().sb200_host_register(self.host.ctypes.data_as(C.c_void_p), self.host.nbytes) == 0:
                self._pinned = True

    def __del__(self):
        if getattr(self, "_prefetch_dev", None) is not None:   # a result still on its way into the array that is going away
            try:
                L.load().sb200_prefetch_wait(self._prefetch_dev)
            except Exception:
                pass
            self._prefetch_dev = None
        if getattr(self, "_pinned", False):     # never leave a registration behind memory that is being released
            try:
                L.load().sb200_host_unregister(self.host.ctypes.data_as(C.c_void_p))
            except Exception:
                pass

    @classmethod
    def create(cls, backend: Backend, n: int) -> "Vector":
        return cls(backend, np.zeros(n, dtype=np.float32))

    @property
    def length(self) -> int:
        return self.host.shape[0]

    def to_device(self, dev: _Device.T) -> None:
        if self.buffer is None:
            self.buffer = self.backend.Memory.alloc(dev, self.length, np.float32)
        if self.location == Vector.CPU:
            self._note_transfer()
            self.backend.Memory.host_to_device(src=self.host, dst=self.buffer)
            self.location = Vector.BOTH

    def pending_upload(self, dev: _Device.T) -> np.ndarray | None:
        """For run_vectors: makes sure the device buffer exists and, when the host copy is the valid one, hands back the
        host array for the launch to upload (the launch call then moves it, overlapped with the kernel where possible)
        instead of copying here; None when the device copy is current."""
        self._finish_prefetch()      # nothing may still be writing the host array when it is read for an upload
        if self.buffer is None:
            self.buffer = self.backend.Memory.alloc(dev, self.length, np.float32)
        if self.location == Vector.CPU:
            self._note_transfer()
            return self.host
        return None

    def _finish_prefetch(self) -> bool:
        if self._prefetch_dev is None:
            return False
        dev, self._prefetch_dev = self._prefetch_dev, None
        _check(L.load().sb200_prefetch_wait(dev))
        return True

    def to_array(self) -> np.ndarray:
        if self._finish_prefetch() and self.location == Vector.STALE_CPU:
            self._note_transfer()
            self.location = Vector.BOTH      # the launch that made the host copy stale has already sent the result back
        if self.location == Vector.STALE_CPU:
            self._note_transfer()
            self.backend.Memory.device_to_host(src=self.buffer, dst=self.host)
            self.location = Vector.BOTH
        return self.host

    def set(self, i: int, v: float) -> None:
        self.to_array()
        self.host[i] = v
        self.location = Vector.CPU

    def free(self) -> None:
        self._finish_prefetch()
        if self._pinned:
            L.load().sb200_host_unregister(self.host.ctypes.data_as(C.c_void_p))
            self._pinned = False
        if self.buffer is not None:
            self.backend.Memory.free(self.buffer)
            self.buffer = None
            if self.location != Vector.CPU:
                self.location = Vector.CPU


def run_vectors(backend: Backend, *, device: _Device.T, ir: str, args: Sequence, block: Dims, grid: Dims,
                shared_mem: int = 0, kernel_name: str = "sarek_kern") -> None:
    """Sarek.Execute.run_vectors: args are Vector objects or ("int32"|"int64"|
    "float32"|"float64", value) pairs in the kernel's parameter order."""
    rs_args = []
    uploaded = []
    prefetch = os.environ.get("SAREK_B200_PREFETCH_RESULTS", "1") != "0"
    for a in args:
        if isinstance(a, Vector):
            # Transfer.to_device of the reference, folded into the launch call so that the library can overlap the two
            host = a.pending_upload(device)
            if host is not None:
                uploaded.append(a)
            # a page-locked host array can take the kernel's result back while later row blocks are still computing
            rs_args.append(RSA_Buffer(a.buffer, a.length, host, a.host if (a._pinned and prefetch) else None))
            rs_args.append(RSA_Int32(a.length))
        else:
            kind, v = a
            rs_args.append({"int32": RSA_Int32, "int64": RSA_Int64, "float32": RSA_Float32, "float64": RSA_Float64}[kind](v))
    backend.Device.set_current(device)
    source = backend.generate_source(ir, block)
    coming_back = backend.run_source(source=source, lang=backend.supported_source_langs[0], kernel_name=kernel_name,
                                     block=block, grid=grid, shared_mem=shared_mem, args=rs_args)
    for i in coming_back:
        vec = next(a for a in args if isinstance(a, Vector) and a.buffer is rs_args[i].buffer)
        vec._prefetch_dev = device.id
    for a in uploaded:   # the launch call returns when its uploads have completed
        a.location = Vector.BOTH
    for a in args:  # mark_vectors_stale
        if isinstance(a, Vector) and a.location == Vector.BOTH:
            a.location = Vector.STALE_CPU
