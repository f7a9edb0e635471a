(** B200_error - the backend's structured errors, built like sarek-cuda/Cuda_error.ml:14-19 from the shared
    functor of spoc/framework/Backend_error.ml, plus the one place where a status of libsarek_b200.so becomes
    one of them.  A Sarek caller that matches on [Backend_error.Backend_error] sees this backend's failures in
    the taxonomy it already handles (spoc/framework/Backend_error.ml:21-78). *)

include Spoc_framework.Backend_error.Make (struct
  let name = "B200"
end)

exception B200_error = Spoc_framework.Backend_error.Backend_error

(** Status codes of include/sb200.h. *)
let err_invalid_value = -1
let err_invalid_handle = -2
let err_unsupported = -3
let err_parse = -4
let err_args = -5
let err_bounds = -6
let err_timeout = -7
let err_no_device = -8
let err_too_large = -9
let err_alignment = -10
let err_comm = -11

(** [of_status ~ctx rc msg]: the error value for a non-zero status. [ctx] is the entry point that returned it
    (or the kernel name for launches), [msg] the library's last error string.
    -3 -> Unsupported_construct (the IR is not a kernel this backend runs; there is no fallback);
    -4 -> Compilation_failed (malformed IR text); -5, -6, -1, -9, -10 -> Kernel_launch_failed (argument list,
    vector bounds, bad value, size beyond a maximum, misalignment: nothing was launched);
    -7 -> Synchronization_failed (a bounded device-side wait expired); -8 -> Backend_unavailable;
    -2 -> Context_error; -11 -> Initialization_failed (NCCL missing or failing);
    positive codes are CUDA runtime errors: 2 (out of memory) -> Memory_allocation_failed, others -> Context_error. *)
let of_status ~ctx rc msg =
  if rc = err_unsupported then unsupported_construct ctx msg
  else if rc = err_parse then compilation_failed ctx msg
  else if rc = err_args || rc = err_bounds || rc = err_invalid_value || rc = err_too_large || rc = err_alignment then
    kernel_launch_failed ctx msg
  else if rc = err_timeout then synchronization_failed msg
  else if rc = err_no_device then backend_unavailable msg
  else if rc = err_invalid_handle then context_error ctx msg
  else if rc = err_comm then initialization_failed msg
  else if rc = 2 then memory_allocation_failed 0L msg
  else context_error ctx (Printf.sprintf "CUDA error %d: %s" rc msg)

let raise_status ~ctx rc msg = raise (B200_error (of_status ~ctx rc msg))
