"""ctypes binding of libsarek_b200.so — the Python twin of the OCaml
``B200_bindings.ml`` a Sarek maintainer would write in the style of
sarek-cuda/Cuda_bindings.ml:39-87 (lazy dlopen + one foreign declaration per
entry point).  No computation happens here; a missing library is an error,
never a fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsarek_b200.so")

# status codes (include/sb200.h)
OK = 0
ERR_INVALID_VALUE, ERR_INVALID_HANDLE, ERR_UNSUPPORTED, ERR_PARSE, ERR_ARGS = -1, -2, -3, -4, -5
ERR_BOUNDS, ERR_TIMEOUT, ERR_NO_DEVICE, ERR_TOO_LARGE, ERR_ALIGNMENT, ERR_COMM = -6, -7, -8, -9, -10, -11
SHARD_GATHER_FUSED, SHARD_GATHER_NCCL, SHARD_B_RESIDENT = 1, 2, 4
MODE_3XTF32, MODE_TF32, MODE_3XF16, MODE_F16, MODE_3XMIXED = 3, 1, 4, 2, 5
ACT_NONE, ACT_RELU = 0, 1
KIND_MAP, KIND_GEMM_NAIVE, KIND_GEMM_TILED, KIND_BLOCK_REDUCE = 1, 2, 3, 4
ARG_BUFFER, ARG_I32, ARG_I64, ARG_F32, ARG_F64 = 0, 1, 2, 3, 4


class ArgValue(C.Union):
    _fields_ = [("buffer", C.c_uint64), ("i32", C.c_int32), ("i64", C.c_int64), ("f32", C.c_float), ("f64", C.c_double)]


class Arg(C.Structure):
    _fields_ = [("tag", C.c_int32), ("reserved", C.c_int32), ("v", ArgValue)]


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("total_mem", C.c_uint64), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("sm_count", C.c_int32), ("max_threads_per_block", C.c_int32), ("max_shared_per_block", C.c_int32),
                ("warp_size", C.c_int32), ("clock_khz", C.c_int32), ("l2_bytes", C.c_int32)]


u64, i64, i32, f32, f64 = C.c_uint64, C.c_int64, C.c_int, C.c_float, C.c_double
p = C.POINTER

# name -> (argtypes, restype); every symbol include/sb200.h declares
SIGNATURES = {
    "sb200_init": ([], i32),
    "sb200_version": ([], i32),
    "sb200_last_error_string": ([], C.c_char_p),
    "sb200_device_count": ([p(i32)], i32),
    "sb200_device_get_info": ([i32, p(DeviceInfo)], i32),
    "sb200_device_set_current": ([i32], i32),
    "sb200_device_synchronize": ([i32], i32),
    "sb200_mem_alloc": ([i32, u64, p(u64)], i32),
    "sb200_mem_free": ([i32, u64], i32),
    "sb200_mem_size": ([i32, u64, p(u64)], i32),
    "sb200_memset32": ([i32, u64, C.c_uint32, u64, u64], i32),
    "sb200_memcpy_htod": ([i32, u64, C.c_void_p, u64], i32),
    "sb200_memcpy_dtoh": ([i32, C.c_void_p, u64, u64], i32),
    "sb200_memcpy_dtod": ([i32, u64, u64, u64], i32),
    "sb200_memcpy_htod_async": ([i32, u64, C.c_void_p, u64, u64], i32),
    "sb200_memcpy_dtoh_async": ([i32, C.c_void_p, u64, u64, u64], i32),
    "sb200_host_alloc": ([u64, p(C.c_void_p)], i32),
    "sb200_host_free": ([C.c_void_p], i32),
    "sb200_host_register": ([C.c_void_p, u64], i32),
    "sb200_host_unregister": ([C.c_void_p], i32),
    "sb200_stream_create": ([i32, p(u64)], i32),
    "sb200_stream_destroy": ([i32, u64], i32),
    "sb200_stream_synchronize": ([i32, u64], i32),
    "sb200_stream_wrap": ([i32, u64, p(u64)], i32),
    "sb200_event_create": ([i32, p(u64)], i32),
    "sb200_event_destroy": ([i32, u64], i32),
    "sb200_event_record": ([i32, u64, u64], i32),
    "sb200_event_synchronize": ([i32, u64], i32),
    "sb200_event_elapsed_ms": ([i32, u64, u64, p(f32)], i32),
    "sb200_kernel_compile": ([i32, C.c_char_p, C.c_char_p, p(u64)], i32),
    "sb200_kernel_destroy": ([u64], i32),
    "sb200_kernel_kind": ([u64, p(i32)], i32),
    "sb200_kernel_describe": ([u64, C.c_char_p, i32], i32),
    "sb200_kernel_launch": ([u64, p(Arg), i32, p(C.c_uint32), p(C.c_uint32), C.c_uint32, u64], i32),
    "sb200_kernel_launch_from_host": ([u64, p(Arg), i32, p(C.c_void_p), p(C.c_void_p), p(C.c_int32), p(C.c_uint32),
                                      p(C.c_uint32), C.c_uint32, u64], i32),
    "sb200_prefetch_wait": ([i32], i32),
    "sb200_ir_can_fuse": ([C.c_char_p, C.c_char_p, C.c_char_p, p(i32)], i32),
    "sb200_ir_fuse": ([C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, i32], i32),
    "sb200_ir_fuse_pipeline": ([p(C.c_char_p), i32, C.c_char_p, i32, C.c_char_p, i32], i32),
    "sb200_ir_fuse_pipeline_as": ([p(C.c_char_p), i32, i32, C.c_char_p, i32, C.c_char_p, i32], i32),
    "sb200_ir_should_fuse": ([C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, i32, C.c_char_p, i32], i32),
    "sb200_ir_auto_fuse_pipeline": ([p(C.c_char_p), i32, C.c_char_p, i32, C.c_char_p, i32, C.c_char_p, i32], i32),
    "sb200_ir_analyze": ([C.c_char_p, C.c_char_p, i32], i32),
    "sb200_ir_can_fuse_as": ([C.c_char_p, C.c_char_p, C.c_char_p, i32, p(i32)], i32),
    "sb200_ir_fuse_as": ([C.c_char_p, C.c_char_p, C.c_char_p, i32, C.c_char_p, i32, p(i32)], i32),
    "sb200_gemm_f32": ([i32, u64, i32, i64, i64, i64, u64, i64, u64, i64, u64, i64, f32, u64, i64, f32, u64, i32], i32),
    "sb200_gemm_f32_noalloc": ([i32, u64, i32, i64, i64, i64, u64, i64, u64, i64, u64, i64, f32, u64, i64, f32, u64, i32], i32),
    "sb200_gemm_f32_gather": ([i32, u64, i32, i64, i64, i64, u64, i64, u64, i64, p(u64), i32, i64, i64, f32, u64, i64, f32, u64, i32], i32),
    "sb200_group_create": ([i32, p(i32), p(u64)], i32),
    "sb200_group_destroy": ([u64], i32),
    "sb200_group_size": ([u64, p(i32)], i32),
    "sb200_group_device": ([u64, i32, p(i32)], i32),
    "sb200_row_block": ([i64, i32, i32, p(i64), p(i64)], i32),
    "sb200_gemm_sharded": ([u64, i32, i64, i64, i64, p(u64), i64, u64, i64, p(u64), i64, f32, p(u64), i64, f32, u64, i32, i32], i32),
    "sb200_group_last_ms": ([u64, p(f32)], i32),
    "sb200_gemm_sharded_host": ([u64, i32, i64, i64, i64, C.c_void_p, i64, C.c_void_p, i64, C.c_void_p, i64, f32, C.c_void_p, i64,
                                 f32, C.c_void_p, i32], i32),
    "sb200_ipc_export": ([i32, u64, C.c_void_p], i32),
    "sb200_ipc_open": ([i32, C.c_void_p, p(u64)], i32),
    "sb200_ipc_close": ([i32, u64], i32),
    "sb200_gemm_f32_host": ([i32, i32, i64, i64, i64, C.c_void_p, i64, C.c_void_p, i64, C.c_void_p, i64, f32, C.c_void_p, i64, f32,
                             C.c_void_p, i32], i32),
    "sb200_gemm_workspace_bytes": ([i32, i64, i64, i64, p(u64)], i32),
    "sb200_vector_add_f32": ([i32, u64, u64, u64, u64, i64], i32),
    "sb200_stream_triad_f32": ([i32, u64, u64, u64, u64, f32, i64], i32),
    "sb200_chain_triad_square_f32": ([i32, u64, u64, u64, u64, u64, f32, i64], i32),
    "sb200_set_mode": ([i32], i32),
    "sb200_get_mode": ([p(i32)], i32),
    "sb200_set_gemm_variant": ([i32], i32),
    "sb200_set_gemm_tile_n": ([i32], i32),
    "sb200_set_lockstep": ([i32], i32),
    "sb200_set_mixed_min_macs": ([i64], i32),
    "sb200_mixed_plan": ([f32, f32, p(C.c_int32)], i32),
    "sb200_set_l2_policy": ([i32], i32),
    "sb200_gemm_describe": ([i32, i64, i64, i64, i32, i32, C.c_char_p, i32], i32),
    "sb200_fill_f32": ([i32, u64, u64, i64, u64, u64, i32, f64, i64], i32),
    "sb200_enable_profiling": ([i32], i32),
    "sb200_profile_gemm_read": ([i32, p(u64), p(f64), p(f64)], i32),
    "sb200_selftest_wait_timeout": ([i32, C.c_uint32], i32),
    "sb200_launch_count": ([p(u64)], i32),
}

_lib = None


class LibraryMissing(RuntimeError):
    pass


def load() -> C.CDLL:
    """dlopen the in-tree library and declare every entry point.  Raises
    LibraryMissing when it has not been built: there is no other code path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m spoc_b200.build` (needs nvcc). "
            "This backend has no CPU or interpreter fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib
