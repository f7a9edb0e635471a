(** B200_plugin - Framework_sig.BACKEND for the B200 backend and its
    registration (the role of sarek-cuda/Cuda_plugin.ml:146-256). *)

open Spoc_framework
open Spoc_framework_registry
module Base = B200_plugin_base.B200

type Framework_sig.kargs += B200_kargs of Base.Kernel.args

(** The thread/block intrinsics are resolved by the library from their names in
    the IR; the registry only has to list them. *)
module B200_intrinsics : Framework_sig.INTRINSIC_REGISTRY = struct
  type intrinsic_impl = {intr_name : string; intr_convergence : Framework_sig.convergence}
  let table : (string, intrinsic_impl) Hashtbl.t = Hashtbl.create 32
  let register n i = Hashtbl.replace table n i
  let find n = Hashtbl.find_opt table n
  let list_all () = Hashtbl.fold (fun n _ acc -> n :: acc) table [] |> List.sort compare
  let () =
    List.iter
      (fun (n, c) -> register n {intr_name = n; intr_convergence = c})
      [ ("thread_idx_x", Framework_sig.Divergent); ("thread_idx_y", Framework_sig.Divergent);
        ("block_idx_x", Framework_sig.Uniform); ("block_idx_y", Framework_sig.Uniform);
        ("block_dim_x", Framework_sig.Uniform); ("block_dim_y", Framework_sig.Uniform);
        ("global_thread_id", Framework_sig.Divergent); ("block_barrier", Framework_sig.Sync) ]
end

module Backend : Framework_sig.BACKEND = struct
  include Base

  (** Set to "CUDA" to take the place of sarek-cuda for every existing caller
      (Framework_registry.register_backend replaces by name). *)
  let name = match Sys.getenv_opt "SAREK_B200_NAME" with Some n -> n | None -> "B200"

  let execution_model = Framework_sig.JIT

  (** The IR text is the backend's source language.  Execute calls this on every launch
      (sarek/sarek/Execute.ml:250-264); the kernel value of a [%kernel] is built once, so the text is cached
      per IR value (physical equality, weak in the key) and a launch re-serialises nothing. *)
  module Ir_cache = Ephemeron.K1.Make (struct
    type t = Sarek_ir_types.kernel
    let equal = ( == )
    let hash (k : t) = Hashtbl.hash k.kern_name
  end)

  let ir_cache : string option Ir_cache.t = Ir_cache.create 16

  let generate_source ?block:_ (ir : Sarek_ir_types.kernel) : string option =
    match Ir_cache.find_opt ir_cache ir with
    | Some s -> s
    | None ->
        let s = try Some (B200_ir_ser.to_sexp ir) with _ -> None in
        Ir_cache.replace ir_cache ir s ;
        s

  let execute_direct ~native_fn:_ ~ir:_ ~block:_ ~grid:_ _args =
    B200_error.raise_error (B200_error.feature_not_supported "execute_direct (this is a JIT backend)")

  module Intrinsics = B200_intrinsics

  (* Execute.run passes the head of this list back as ~lang; the text is not CUDA C,
     the tag only routes the call to run_source below. *)
  let supported_source_langs = [Framework_sig.CUDA_Source]

  let run_source ~source ~lang:_ ~kernel_name ~block ~grid ~shared_mem args =
    let dev =
      match Device.get_current_device () with
      | Some d -> d
      | None -> B200_error.raise_error (B200_error.no_device_selected "run_source")
    in
    let compiled = Kernel.compile_cached dev ~name:kernel_name ~source in
    let kargs = Kernel.create_args () in
    let wrapped = B200_kargs kargs in
    List.iteri
      (fun i arg ->
        match arg with
        | Framework_sig.RSA_Buffer {binder; _} -> binder wrapped i
        | Framework_sig.RSA_Int32 n -> Kernel.set_arg_int32 kargs i n
        | Framework_sig.RSA_Int64 n -> Kernel.set_arg_int64 kargs i n
        | Framework_sig.RSA_Float32 f -> Kernel.set_arg_float32 kargs i f
        | Framework_sig.RSA_Float64 f -> Kernel.set_arg_float64 kargs i f)
      args ;
    Kernel.launch compiled ~args:kargs ~grid ~block ~shared_mem ~stream:(Some (Stream.default dev))

  let wrap_kargs a = B200_kargs a
  let unwrap_kargs = function B200_kargs a -> Some a | _ -> None
end

(** The backend's guarded fusion: [Some text] is the fused kernel in the text form [run_source]
    takes (pass it as [~source] with the merged argument list: the consumer's arguments without the
    intermediate, then the producer's that are new by name), [None] when a condition fails — the
    library's last error string then names it.  Covers the kernel form of the benchmarks,
    [let tid = global_thread_id in if tid < n then ...], which [Sarek_fusion.fuse] gives back
    unfused (sarek/sarek/Sarek_fusion.ml:370-375). *)
let fuse_guarded (producer : Sarek_ir_types.kernel) (consumer : Sarek_ir_types.kernel) (intermediate : string) :
    string option =
  let open Ctypes in
  let len = 1 lsl 20 in
  let buf = allocate_n char ~count:len in
  let fused = allocate int 0 in
  B200_bindings.check "sb200_ir_fuse_as"
    (Lazy.force B200_bindings.sb200_ir_fuse_as
       (B200_ir_ser.to_sexp producer) (B200_ir_ser.to_sexp consumer) intermediate 5 buf len fused) ;
  if !@fused = 0 then None else Some (Ctypes.coerce (ptr char) string buf)

let is_disabled () =
  Sys.getenv_opt "SPOC_DISABLE_GPU" = Some "1" || Sys.getenv_opt "SPOC_DISABLE_B200" = Some "1"

(* priority above sarek-cuda's 100 *)
let registered_backend =
  lazy
    (if Backend.is_available () then
       Framework_registry.register_backend ~priority:110 (module Backend : Framework_sig.BACKEND))

let () = if not (is_disabled ()) then Lazy.force registered_backend
let init () = if not (is_disabled ()) then Lazy.force registered_backend
