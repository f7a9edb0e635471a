"""Sarek_fusion's interface (sarek/sarek/Sarek_fusion.ml) over the library's IR-text
implementation: analyze, can_fuse, fuse, fuse_pipeline, should_fuse, auto_fuse_pipeline."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

from . import _lib as L
from .plugin import _check

_BUF = 1 << 20


def _arr(kernels: Sequence[str]):
    enc = [k.encode() for k in kernels]
    return (C.c_char_p * len(enc))(*enc), len(enc)


def analyze(kernel: str) -> dict:
    """{"reads": {array: pattern}, "writes": {array: pattern}, "has_barriers": bool}."""
    out = C.create_string_buffer(_BUF)
    _check(L.load().sb200_ir_analyze(kernel.encode(), out, _BUF))
    info = {"reads": {}, "writes": {}, "has_barriers": False}
    for line in out.value.decode().splitlines():
        f = line.split()
        if f[0] == "barriers":
            info["has_barriers"] = f[1] == "yes"
        else:
            info["reads" if f[0] == "read" else "writes"][f[1]] = f[2]
    return info


def can_fuse(producer: str, consumer: str, intermediate: str) -> bool:
    r = C.c_int(0)
    _check(L.load().sb200_ir_can_fuse(producer.encode(), consumer.encode(), intermediate.encode(), C.byref(r)))
    return bool(r.value)


def fuse(producer: str, consumer: str, intermediate: str) -> str:
    out = C.create_string_buffer(_BUF)
    _check(L.load().sb200_ir_fuse(producer.encode(), consumer.encode(), intermediate.encode(), out, _BUF))
    return out.value.decode()


def fuse_pipeline(kernels: Sequence[str]) -> tuple[str, list[str]]:
    arr, n = _arr(kernels)
    out, elim = C.create_string_buffer(_BUF), C.create_string_buffer(4096)
    _check(L.load().sb200_ir_fuse_pipeline(arr, n, out, _BUF, elim, 4096))
    e = elim.value.decode()
    return out.value.decode(), (e.split(",") if e else [])


def should_fuse(producer: str, consumer: str, intermediate: str) -> tuple[str, str]:
    d, r = C.create_string_buffer(64), C.create_string_buffer(256)
    _check(L.load().sb200_ir_should_fuse(producer.encode(), consumer.encode(), intermediate.encode(), d, 64, r, 256))
    return d.value.decode(), r.value.decode()


def auto_fuse_pipeline(kernels: Sequence[str]) -> tuple[str, list[str], list[str]]:
    arr, n = _arr(kernels)
    out, elim, skip = C.create_string_buffer(_BUF), C.create_string_buffer(4096), C.create_string_buffer(8192)
    _check(L.load().sb200_ir_auto_fuse_pipeline(arr, n, out, _BUF, elim, 4096, skip, 8192))
    e, s = elim.value.decode(), skip.value.decode()
    return out.value.decode(), (e.split(",") if e else []), (s.split("\n") if s else [])


PLAIN, REDUCTION, STENCIL, TRY, TRY_ALL, GUARDED = 0, 1, 2, 3, 4, 5


def _can_as(producer: str, consumer: str, intermediate: str, kind: int) -> bool:
    r = C.c_int(0)
    _check(L.load().sb200_ir_can_fuse_as(producer.encode(), consumer.encode(), intermediate.encode(), kind, C.byref(r)))
    return bool(r.value)


def _fuse_as(producer: str, consumer: str, intermediate: str, kind: int):
    out, f = C.create_string_buffer(_BUF), C.c_int(0)
    _check(L.load().sb200_ir_fuse_as(producer.encode(), consumer.encode(), intermediate.encode(), kind, out, _BUF, C.byref(f)))
    return out.value.decode() if f.value else None


def can_fuse_reduction(map_kernel: str, reduce_kernel: str, intermediate: str) -> bool:
    return _can_as(map_kernel, reduce_kernel, intermediate, REDUCTION)


def fuse_reduction(map_kernel: str, reduce_kernel: str, intermediate: str) -> str:
    return _fuse_as(map_kernel, reduce_kernel, intermediate, REDUCTION)


def can_fuse_stencil(producer: str, consumer: str, intermediate: str) -> bool:
    return _can_as(producer, consumer, intermediate, STENCIL)


def fuse_stencil(producer: str, consumer: str, intermediate: str) -> str:
    return _fuse_as(producer, consumer, intermediate, STENCIL)


def try_fuse(producer: str, consumer: str, intermediate: str):
    """Fused kernel text, or None (the reference's `kernel option`)."""
    return _fuse_as(producer, consumer, intermediate, TRY)


def try_fuse_all(producer: str, consumer: str, intermediate: str):
    return _fuse_as(producer, consumer, intermediate, TRY_ALL)


def can_fuse_guarded(producer: str, consumer: str, intermediate: str) -> bool:
    """This backend's extension (not in the reference): kernels of the guarded form
    ``let tid = global_thread_id in if tid < n then out.(tid) <- e`` — the form of the reference's own
    benchmark kernels, which its pass leaves unfused (sarek/sarek/Sarek_fusion.ml:370-375)."""
    return _can_as(producer, consumer, intermediate, GUARDED)


def fuse_guarded(producer: str, consumer: str, intermediate: str):
    """Fused kernel text, or None; ``why_not_fused()`` then names the failed condition."""
    return _fuse_as(producer, consumer, intermediate, GUARDED)


def why_not_fused() -> str:
    return L.load().sb200_last_error_string().decode()


def fuse_pipeline_as(kernels: Sequence[str], kind: int) -> tuple[str, list[str]]:
    """fuse_pipeline with the fusion form of each step chosen by ``kind`` (PLAIN ... GUARDED)."""
    arr, n = _arr(kernels)
    out, elim = C.create_string_buffer(_BUF), C.create_string_buffer(4096)
    _check(L.load().sb200_ir_fuse_pipeline_as(arr, n, kind, out, _BUF, elim, 4096))
    e = elim.value.decode()
    return out.value.decode(), (e.split(",") if e else [])
