(** B200_group - several GPUs of this process as one object (include/sb200.h: device groups).

    Sarek's multi-device model is to partition a vector and launch once per device
    (sarek/core/Vector.ml:273-296; split rule sarek/core/Vector_storage.ml:261-272).  For the matmul path the library
    does that inside one call: B crosses PCIe once and reaches the other GPUs by NCCL broadcast, every GPU moves and
    computes its own row block of A, C and D.  [gemm_host] is what a caller with Bigarray-backed vectors uses;
    [gemm] takes row shards that already live on the members' GPUs ([Memory.alloc] on each member device). *)

open Ctypes
module B = B200_bindings

type t = {handle : Unsigned.UInt64.t; devices : int list}

type gather = No_gather | Gather_fused | Gather_nccl

(** 1 to 8 distinct device indices; raises [Backend_error] (Kernel_launch_failed for a bad list,
    Initialization_failed when NCCL cannot be loaded). *)
let create (devices : int list) : t =
  let n = List.length devices in
  let arr = CArray.of_list int devices in
  let h = allocate uint64_t Unsigned.UInt64.zero in
  B.check "sb200_group_create" (Lazy.force B.sb200_group_create n (CArray.start arr) h) ;
  {handle = !@h; devices}

let destroy g = B.check "sb200_group_destroy" (Lazy.force B.sb200_group_destroy g.handle)
let size g = List.length g.devices

(** [(first, rows)] of member [i] when [m] rows are split over the group: the reference's partition rule. *)
let row_block g m i =
  let first = allocate int64_t 0L and rows = allocate int64_t 0L in
  B.check "sb200_row_block" (Lazy.force B.sb200_row_block (Int64.of_int m) (size g) i first rows) ;
  (Int64.to_int !@first, Int64.to_int !@rows)

let mode_code = function `X3_tf32 -> 3 | `Tf32 -> 1 | `X3_f16 -> 4 | `F16 -> 2

type f32_array = (float, Bigarray.float32_elt, Bigarray.c_layout) Bigarray.Array1.t

let ptr_of (a : f32_array) = bigarray_start array1 a
let opt_ptr = function Some a -> ptr_of a | None -> from_voidp float null

(** D = act(alpha * A.B + beta * C + bias) on host operands (row-major, contiguous); D is written in place. *)
let gemm_host g ?(mode = `X3_tf32) ~m ~n ~k ~(a : f32_array) ~(b : f32_array) ~(d : f32_array) ?(alpha = 1.0) ?c ?(beta = 0.0)
    ?bias ?(relu = false) () =
  let i64 = Int64.of_int in
  B.check "sb200_gemm_sharded_host"
    (Lazy.force B.sb200_gemm_sharded_host g.handle (mode_code mode) (i64 m) (i64 n) (i64 k) (ptr_of a) (i64 k) (ptr_of b) (i64 n)
       (ptr_of d) (i64 n) alpha (opt_ptr c) (i64 n) beta (opt_ptr bias) (if relu then 1 else 0))

(** The same on device-resident row shards: [a_shards], [c_shards] and [d] hold one device pointer per member
    ([d] whole copies of D when [gather] is not [No_gather]); [b] and [bias] lie on the first member's GPU. *)
let gemm g ?(mode = `X3_tf32) ~m ~n ~k ~(a_shards : Unsigned.UInt64.t list) ~(b : Unsigned.UInt64.t) ~(d : Unsigned.UInt64.t list)
    ?(alpha = 1.0) ?c_shards ?(beta = 0.0) ?(bias = Unsigned.UInt64.zero) ?(relu = false) ?(gather = No_gather) ?(b_resident = false) () =
  let i64 = Int64.of_int in
  let tab l = CArray.start (CArray.of_list uint64_t l) in
  let flags = (match gather with No_gather -> 0 | Gather_fused -> 1 | Gather_nccl -> 2) lor if b_resident then 4 else 0 in
  let c_tab = match c_shards with Some l -> tab l | None -> from_voidp uint64_t null in
  B.check "sb200_gemm_sharded"
    (Lazy.force B.sb200_gemm_sharded g.handle (mode_code mode) (i64 m) (i64 n) (i64 k) (tab a_shards) (i64 k) b (i64 n) (tab d) (i64 n)
       alpha c_tab (i64 n) beta bias (if relu then 1 else 0) flags)
