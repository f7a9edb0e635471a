(** B200_bindings - ctypes-foreign bindings to libsarek_b200.so, in the style of
    sarek-cuda/Cuda_bindings.ml: the library is opened lazily and every entry
    point is a lazy foreign value. All functions return an int status. *)

open Ctypes
open Foreign

let lib : Dl.library option Lazy.t =
  lazy
    (let try_open f = try Some (Dl.dlopen ~filename:f ~flags:[Dl.RTLD_LAZY; Dl.RTLD_GLOBAL]) with _ -> None in
     match try_open "libsarek_b200.so" with
     | Some l -> Some l
     | None -> (
         match Sys.getenv_opt "SAREK_B200_LIB" with Some p -> try_open p | None -> None))

let is_available () = match Lazy.force lib with Some _ -> true | None -> false

let get () =
  match Lazy.force lib with
  | Some l -> l
  | None -> B200_error.raise_error (B200_error.library_not_found "libsarek_b200.so" ["LD_LIBRARY_PATH"; "SAREK_B200_LIB"])

let fn name typ = lazy (foreign ~from:(get ()) name typ)

(* struct sb200_arg { int32 tag; int32 reserved; union { u64; i32; i64; f32; f64 } v; } : 16 bytes *)
type sb200_arg
let sb200_arg : sb200_arg structure typ = structure "sb200_arg"
let arg_tag = field sb200_arg "tag" int32_t
let _arg_reserved = field sb200_arg "reserved" int32_t
let arg_value = field sb200_arg "v" uint64_t (* every member of the union fits in, and is read from, these 8 bytes *)
let () = seal sb200_arg

(* struct sb200_device_info *)
type device_info
let device_info : device_info structure typ = structure "sb200_device_info"
let di_name = field device_info "name" (array 256 char)
let di_total_mem = field device_info "total_mem" uint64_t
let di_cc_major = field device_info "cc_major" int32_t
let di_cc_minor = field device_info "cc_minor" int32_t
let di_sm_count = field device_info "sm_count" int32_t
let di_max_threads = field device_info "max_threads_per_block" int32_t
let di_max_shared = field device_info "max_shared_per_block" int32_t
let di_warp_size = field device_info "warp_size" int32_t
let di_clock_khz = field device_info "clock_khz" int32_t
let di_l2_bytes = field device_info "l2_bytes" int32_t
let () = seal device_info

let sb200_init = fn "sb200_init" (void @-> returning int)
let sb200_last_error_string = fn "sb200_last_error_string" (void @-> returning string)
let sb200_device_count = fn "sb200_device_count" (ptr int @-> returning int)
let sb200_device_get_info = fn "sb200_device_get_info" (int @-> ptr device_info @-> returning int)
let sb200_device_set_current = fn "sb200_device_set_current" (int @-> returning int)
let sb200_device_synchronize = fn "sb200_device_synchronize" (int @-> returning int)
let sb200_mem_alloc = fn "sb200_mem_alloc" (int @-> uint64_t @-> ptr uint64_t @-> returning int)
let sb200_mem_free = fn "sb200_mem_free" (int @-> uint64_t @-> returning int)
let sb200_memcpy_htod = fn "sb200_memcpy_htod" (int @-> uint64_t @-> ptr void @-> uint64_t @-> returning int)
let sb200_memcpy_dtoh = fn "sb200_memcpy_dtoh" (int @-> ptr void @-> uint64_t @-> uint64_t @-> returning int)
let sb200_memcpy_dtod = fn "sb200_memcpy_dtod" (int @-> uint64_t @-> uint64_t @-> uint64_t @-> returning int)
let sb200_host_register = fn "sb200_host_register" (ptr void @-> uint64_t @-> returning int)
let sb200_host_unregister = fn "sb200_host_unregister" (ptr void @-> returning int)
let sb200_stream_create = fn "sb200_stream_create" (int @-> ptr uint64_t @-> returning int)
let sb200_stream_destroy = fn "sb200_stream_destroy" (int @-> uint64_t @-> returning int)
let sb200_stream_synchronize = fn "sb200_stream_synchronize" (int @-> uint64_t @-> returning int)
let sb200_event_create = fn "sb200_event_create" (int @-> ptr uint64_t @-> returning int)
let sb200_event_destroy = fn "sb200_event_destroy" (int @-> uint64_t @-> returning int)
let sb200_event_record = fn "sb200_event_record" (int @-> uint64_t @-> uint64_t @-> returning int)
let sb200_event_synchronize = fn "sb200_event_synchronize" (int @-> uint64_t @-> returning int)
let sb200_event_elapsed_ms = fn "sb200_event_elapsed_ms" (int @-> uint64_t @-> uint64_t @-> ptr float @-> returning int)
let sb200_kernel_compile = fn "sb200_kernel_compile" (int @-> string @-> string @-> ptr uint64_t @-> returning int)
let sb200_kernel_destroy = fn "sb200_kernel_destroy" (uint64_t @-> returning int)
let sb200_kernel_launch =
  fn "sb200_kernel_launch"
    (uint64_t @-> ptr sb200_arg @-> int @-> ptr uint32_t @-> ptr uint32_t @-> uint32_t @-> uint64_t @-> returning int)
(* upload + launch (+ result sent back) in one call; see B200_plugin_base.Deferred *)
let sb200_kernel_launch_from_host =
  fn "sb200_kernel_launch_from_host"
    (uint64_t @-> ptr sb200_arg @-> int @-> ptr (ptr void) @-> ptr (ptr void) @-> ptr int32_t @-> ptr uint32_t
   @-> ptr uint32_t @-> uint32_t @-> uint64_t @-> returning int)
let sb200_prefetch_wait = fn "sb200_prefetch_wait" (int @-> returning int)
let sb200_enable_profiling = fn "sb200_enable_profiling" (int @-> returning int)
let sb200_set_mode = fn "sb200_set_mode" (int @-> returning int)
let sb200_set_lockstep = fn "sb200_set_lockstep" (int @-> returning int)
(* fusion on IR text; kind 5 = the backend's guarded fusion of `if tid < n then ..` kernels,
   which Sarek_fusion leaves unfused (sarek/sarek/Sarek_fusion.ml:370-375) *)
let sb200_ir_fuse_as =
  fn "sb200_ir_fuse_as" (string @-> string @-> string @-> int @-> ptr char @-> int @-> ptr int @-> returning int)

(* one process, several GPUs (include/sb200.h: device groups) *)
let sb200_group_create = fn "sb200_group_create" (int @-> ptr int @-> ptr uint64_t @-> returning int)
let sb200_group_destroy = fn "sb200_group_destroy" (uint64_t @-> returning int)
let sb200_row_block = fn "sb200_row_block" (int64_t @-> int @-> int @-> ptr int64_t @-> ptr int64_t @-> returning int)
let sb200_gemm_sharded =
  fn "sb200_gemm_sharded"
    (uint64_t @-> int @-> int64_t @-> int64_t @-> int64_t @-> ptr uint64_t @-> int64_t @-> uint64_t @-> int64_t
   @-> ptr uint64_t @-> int64_t @-> float @-> ptr uint64_t @-> int64_t @-> float @-> uint64_t @-> int @-> int
   @-> returning int)
let sb200_gemm_sharded_host =
  fn "sb200_gemm_sharded_host"
    (uint64_t @-> int @-> int64_t @-> int64_t @-> int64_t @-> ptr float @-> int64_t @-> ptr float @-> int64_t
   @-> ptr float @-> int64_t @-> float @-> ptr float @-> int64_t @-> float @-> ptr float @-> int @-> returning int)

(** Non-zero status -> [Backend_error.Backend_error] (see B200_error.of_status for the mapping: -3 is
    Unsupported_construct, -4 Compilation_failed, -5/-6 Kernel_launch_failed, -7 Synchronization_failed, ...),
    carrying the library's message. *)
let check ctx rc =
  if rc <> 0 then B200_error.raise_status ~ctx rc (Lazy.force sb200_last_error_string ())
