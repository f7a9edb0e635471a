(** B200_plugin_base - Device / Stream / Memory / Event / Kernel of
    Framework_sig.BACKEND over the bindings (the role of
    sarek-cuda/Cuda_plugin_base.ml). *)

open Ctypes
open Spoc_framework
module B = B200_bindings

module B200 = struct
  let name = "B200"
  let version = (1, 0, 0)

  let is_available () =
    B.is_available ()
    &&
    let n = allocate int 0 in
    Lazy.force B.sb200_device_count n = 0 && !@n > 0

  (* Launch from host (opt-in: SAREK_B200_LAUNCH_FROM_HOST=1).  Execute.run_vectors moves every vector with
     Transfer.to_device and then launches (sarek/sarek/Execute.ml:520-543); the library can overlap the two when it is
     given both in one call (sb200_kernel_launch_from_host).  With the switch on, Memory.host_to_device from a Bigarray
     that is already registered with the driver only records the upload; the next launch that binds the buffer hands
     the host address to the library, and anything else that touches the buffer (a download, a device copy, a
     synchronize) carries the recorded upload out first.  The launch also names the registered array of every buffer
     argument as the place its result may be sent back to; Memory.device_to_host into that same array then only waits.
     The one observable difference, and the reason for the switch: a Bigarray written behind the vector's back between
     to_device and the launch is uploaded with its new contents. *)
  module Deferred = struct
    let enabled = lazy (Sys.getenv_opt "SAREK_B200_LAUNCH_FROM_HOST" = Some "1")

    type upload = {dev : int; host : unit ptr; bytes : int; keep : Obj.t (* the Bigarray, kept alive *)}

    let key (dptr : Unsigned.UInt64.t) = Unsigned.UInt64.to_int64 dptr
    let uploads : (int64, Unsigned.UInt64.t * upload) Hashtbl.t = Hashtbl.create 16
    let host_copy : (int64, unit ptr) Hashtbl.t = Hashtbl.create 16

    (* device buffer -> (device, host address the result goes to, true once it has arrived) *)
    let results : (int64, int * nativeint * bool) Hashtbl.t = Hashtbl.create 16

    let flush dptr =
      match Hashtbl.find_opt uploads (key dptr) with
      | None -> ()
      | Some (_, u) ->
          Hashtbl.remove uploads (key dptr) ;
          B.check "sb200_memcpy_htod"
            (Lazy.force B.sb200_memcpy_htod u.dev dptr u.host (Unsigned.UInt64.of_int u.bytes))

    let flush_all () = List.iter flush (Hashtbl.fold (fun _ (dptr, _) acc -> dptr :: acc) uploads [])

    let wait_results dev =
      if Hashtbl.fold (fun _ (d, _, arrived) acc -> acc || (d = dev && not arrived)) results false then begin
        B.check "sb200_prefetch_wait" (Lazy.force B.sb200_prefetch_wait dev) ;
        Hashtbl.filter_map_inplace (fun _ (d, h, a) -> Some (d, h, a || d = dev)) results
      end

    let forget dptr =
      Hashtbl.remove uploads (key dptr) ;
      Hashtbl.remove host_copy (key dptr) ;
      Hashtbl.remove results (key dptr)
  end

  module Device = struct
    type t = {idx : int; dev_name : string; caps : Framework_sig.capabilities}
    type id = int

    let current : t option ref = ref None
    let init () = B.check "sb200_init" (Lazy.force B.sb200_init ())

    let count () =
      let n = allocate int 0 in
      B.check "sb200_device_count" (Lazy.force B.sb200_device_count n) ;
      !@n

    let get idx =
      let info = make B.device_info in
      B.check "sb200_device_get_info" (Lazy.force B.sb200_device_get_info idx (addr info)) ;
      let i32 f = Int32.to_int (getf info f) in
      let name_chars = CArray.to_list (getf info B.di_name) in
      let buf = Buffer.create 64 in
      (try List.iter (fun c -> if c = '\000' then raise Exit else Buffer.add_char buf c) name_chars with Exit -> ()) ;
      {
        idx;
        dev_name = Buffer.contents buf;
        caps =
          {
            Framework_sig.max_threads_per_block = i32 B.di_max_threads;
            max_block_dims = (1024, 1024, 64);
            max_grid_dims = (2147483647, 65535, 65535);
            shared_mem_per_block = i32 B.di_max_shared;
            total_global_mem = Unsigned.UInt64.to_int64 (getf info B.di_total_mem);
            compute_capability = (i32 B.di_cc_major, i32 B.di_cc_minor);
            supports_fp64 = true;
            supports_atomics = true;
            warp_size = i32 B.di_warp_size;
            max_registers_per_block = 65536;
            clock_rate_khz = i32 B.di_clock_khz;
            multiprocessor_count = i32 B.di_sm_count;
            is_cpu = false;
          };
      }

    let id d = d.idx
    let name d = d.dev_name
    let capabilities d = d.caps

    let set_current d =
      B.check "sb200_device_set_current" (Lazy.force B.sb200_device_set_current d.idx) ;
      current := Some d

    let get_current_device () = !current
    let synchronize d =
      Deferred.flush_all () ;
      B.check "sb200_device_synchronize" (Lazy.force B.sb200_device_synchronize d.idx)
  end

  module Stream = struct
    type t = {dev : int; handle : Unsigned.UInt64.t}

    let create (d : Device.t) =
      let h = allocate uint64_t Unsigned.UInt64.zero in
      B.check "sb200_stream_create" (Lazy.force B.sb200_stream_create d.idx h) ;
      {dev = d.idx; handle = !@h}

    let destroy s = B.check "sb200_stream_destroy" (Lazy.force B.sb200_stream_destroy s.dev s.handle)
    let synchronize s =
      Deferred.flush_all () ;
      B.check "sb200_stream_synchronize" (Lazy.force B.sb200_stream_synchronize s.dev s.handle)
    let default (d : Device.t) = {dev = d.idx; handle = Unsigned.UInt64.zero}
  end

  module Memory = struct
    type 'a buffer = {dev : int; dptr : Unsigned.UInt64.t; elems : int; elem_size : int}

    let alloc_custom (d : Device.t) ~size ~elem_size =
      let p = allocate uint64_t Unsigned.UInt64.zero in
      B.check "sb200_mem_alloc"
        (Lazy.force B.sb200_mem_alloc d.idx (Unsigned.UInt64.of_int (size * elem_size)) p) ;
      {dev = d.idx; dptr = !@p; elems = size; elem_size}

    let alloc d size kind = alloc_custom d ~size ~elem_size:(Bigarray.kind_size_in_bytes kind)
    let alloc_zero_copy _ _ _ = None

    (* idempotent in the library: a GC finaliser may call it a second time *)
    let free b =
      (match Hashtbl.find_opt Deferred.results (Deferred.key b.dptr) with
      | Some (dev, _, false) -> Deferred.wait_results dev
      | _ -> ()) ;
      Deferred.forget b.dptr ;
      B.check "sb200_mem_free" (Lazy.force B.sb200_mem_free b.dev b.dptr)

    let host_ptr_to_device ~src_ptr ~byte_size ~dst =
      B.check "sb200_memcpy_htod"
        (Lazy.force B.sb200_memcpy_htod dst.dev dst.dptr src_ptr (Unsigned.UInt64.of_int byte_size))

    let device_to_host_ptr ~src ~dst_ptr ~byte_size =
      B.check "sb200_memcpy_dtoh"
        (Lazy.force B.sb200_memcpy_dtoh src.dev dst_ptr src.dptr (Unsigned.UInt64.of_int byte_size))

    (* A Bigarray's storage does not move and lives as long as the Bigarray, so it can be pinned in place.  The first
       transfer of a Bigarray goes through the library's staged pageable copier; one of 16 MiB or more that is moved a
       second time is registered with the driver (sb200_host_register), after which this and every later transfer run
       at the pinned rate.  A finaliser on the Bigarray unregisters before its storage is released.
       SAREK_B200_PIN_VECTORS=0 switches this off. *)
    let pin_threshold = 16 * 1024 * 1024
    let pin_enabled = lazy (Sys.getenv_opt "SAREK_B200_PIN_VECTORS" <> Some "0")
    let seen : (nativeint, int) Hashtbl.t = Hashtbl.create 64
    let registered : (nativeint, unit) Hashtbl.t = Hashtbl.create 64

    let note_transfer (type a b) (ba : (a, b, Bigarray.c_layout) Bigarray.Array1.t) bytes =
      if bytes >= pin_threshold && Lazy.force pin_enabled then begin
        let p = bigarray_start array1 ba in
        let key = raw_address_of_ptr (to_voidp p) in
        let n = 1 + Option.value ~default:0 (Hashtbl.find_opt seen key) in
        Hashtbl.replace seen key n ;
        if n = 2 && Lazy.force B.sb200_host_register (to_voidp p) (Unsigned.UInt64.of_int bytes) = 0 then begin
          Hashtbl.replace registered key () ;
          Gc.finalise
            (fun ba ->
              let p = to_voidp (bigarray_start array1 ba) in
              Hashtbl.remove seen (raw_address_of_ptr p) ;
              Hashtbl.remove registered (raw_address_of_ptr p) ;
              ignore (Lazy.force B.sb200_host_unregister p))
            ba
        end
      end

    let host_to_device ~src ~dst =
      let bytes = Bigarray.Array1.dim src * Bigarray.kind_size_in_bytes (Bigarray.Array1.kind src) in
      note_transfer src bytes ;
      let p = to_voidp (bigarray_start array1 src) in
      Hashtbl.remove Deferred.results (Deferred.key dst.dptr) ;
      if Lazy.force Deferred.enabled && bytes = dst.elems * dst.elem_size && Hashtbl.mem registered (raw_address_of_ptr p) then begin
        (* recorded, carried out by the next launch that binds dst (or by whatever touches dst first) *)
        Hashtbl.replace Deferred.uploads (Deferred.key dst.dptr) (dst.dptr, {Deferred.dev = dst.dev; host = p; bytes; keep = Obj.repr src}) ;
        Hashtbl.replace Deferred.host_copy (Deferred.key dst.dptr) p
      end
      else begin
        Hashtbl.remove Deferred.uploads (Deferred.key dst.dptr) ;
        host_ptr_to_device ~src_ptr:p ~byte_size:bytes ~dst
      end

    let device_to_host ~src ~dst =
      let bytes = Bigarray.Array1.dim dst * Bigarray.kind_size_in_bytes (Bigarray.Array1.kind dst) in
      note_transfer dst bytes ;
      let p = to_voidp (bigarray_start array1 dst) in
      Deferred.flush src.dptr ;
      (match Hashtbl.find_opt Deferred.results (Deferred.key src.dptr) with
      | Some (dev, _, false) -> Deferred.wait_results dev
      | _ -> ()) ;
      match Hashtbl.find_opt Deferred.results (Deferred.key src.dptr) with
      | Some (_, host, true) when host = raw_address_of_ptr p && bytes = src.elems * src.elem_size ->
          (* the launch that wrote src has already sent it back to this very array; good for one read *)
          Hashtbl.remove Deferred.results (Deferred.key src.dptr)
      | _ ->
          if Lazy.force Deferred.enabled && Hashtbl.mem registered (raw_address_of_ptr p) then
            Hashtbl.replace Deferred.host_copy (Deferred.key src.dptr) p ;
          device_to_host_ptr ~src ~dst_ptr:p ~byte_size:bytes

    let device_to_device ~src ~dst =
      Deferred.flush src.dptr ;
      Deferred.forget dst.dptr ;
      let bytes = min (src.elems * src.elem_size) (dst.elems * dst.elem_size) in
      B.check "sb200_memcpy_dtod"
        (Lazy.force B.sb200_memcpy_dtod dst.dev dst.dptr src.dptr (Unsigned.UInt64.of_int bytes))

    let size b = b.elems
    let device_ptr b = Nativeint.of_string (Unsigned.UInt64.to_string b.dptr)
    let is_zero_copy _ = false
  end

  module Event = struct
    type t = {dev : int; handle : Unsigned.UInt64.t}

    let create () =
      let dev = match !Device.current with Some d -> d.idx | None -> 0 in
      let h = allocate uint64_t Unsigned.UInt64.zero in
      B.check "sb200_event_create" (Lazy.force B.sb200_event_create dev h) ;
      {dev; handle = !@h}

    let destroy e = B.check "sb200_event_destroy" (Lazy.force B.sb200_event_destroy e.dev e.handle)
    let record e (s : Stream.t) = B.check "sb200_event_record" (Lazy.force B.sb200_event_record e.dev e.handle s.handle)
    let synchronize e = B.check "sb200_event_synchronize" (Lazy.force B.sb200_event_synchronize e.dev e.handle)

    let elapsed ~start ~stop =
      let ms = allocate float 0.0 in
      B.check "sb200_event_elapsed_ms" (Lazy.force B.sb200_event_elapsed_ms start.dev start.handle stop.handle ms) ;
      !@ms
  end

  module Kernel = struct
    type t = {dev : int; handle : Unsigned.UInt64.t}

    (* positional list, newest first; set_arg_* ignore their index and append,
       like sarek-cuda/Cuda_plugin_base.ml:268-281 *)
    type arg = A_buffer of Unsigned.UInt64.t | A_i32 of int32 | A_i64 of int64 | A_f32 of float | A_f64 of float
    type args = {mutable items : arg list}

    let cache : (int * string, t) Hashtbl.t = Hashtbl.create 16

    (* Launch path: Execute hands run_source the string that generate_source returned, and generate_source
       returns the same string object for the same IR value (B200_plugin.generate_source caches by physical
       equality).  So the common case is a lookup by the string's identity, with no digest of the text; the
       digest-keyed table is the reference's own caching level (sarek-cuda/Cuda_api.ml:399-412) behind it. *)
    module By_identity = Ephemeron.K1.Make (struct
      type t = string
      let equal = ( == )
      let hash s = Hashtbl.hash (String.length s)
    end)

    let by_identity : (int * t) list By_identity.t = By_identity.create 16

    let compile (d : Device.t) ~name ~source =
      let h = allocate uint64_t Unsigned.UInt64.zero in
      B.check "sb200_kernel_compile" (Lazy.force B.sb200_kernel_compile d.idx source name h) ;
      {dev = d.idx; handle = !@h}

    let compile_cached (d : Device.t) ~name ~source =
      let known = match By_identity.find_opt by_identity source with Some l -> l | None -> [] in
      match List.assoc_opt d.idx known with
      | Some k -> k
      | None ->
          let key = (d.idx, Digest.string source) in
          let k =
            match Hashtbl.find_opt cache key with
            | Some k -> k
            | None ->
                let k = compile d ~name ~source in
                Hashtbl.replace cache key k ;
                k
          in
          By_identity.replace by_identity source ((d.idx, k) :: known) ;
          k

    let clear_cache () =
      Hashtbl.iter (fun _ k -> ignore (Lazy.force B.sb200_kernel_destroy k.handle)) cache ;
      Hashtbl.reset cache ;
      By_identity.reset by_identity

    let create_args () = {items = []}
    let push a x = a.items <- x :: a.items
    let set_arg_buffer a _ (b : _ Memory.buffer) = push a (A_buffer b.dptr)
    let set_arg_ptr a _ p = push a (A_buffer (Unsigned.UInt64.of_string (Nativeint.to_string p)))
    let set_arg_int32 a _ v = push a (A_i32 v)
    let set_arg_int64 a _ v = push a (A_i64 v)
    let set_arg_float32 a _ v = push a (A_f32 v)
    let set_arg_float64 a _ v = push a (A_f64 v)

    let launch k ~args ~(grid : Framework_sig.dims) ~(block : Framework_sig.dims) ~shared_mem ~(stream : Stream.t option) =
      let items = List.rev args.items in
      let n = List.length items in
      let arr = CArray.make B.sb200_arg (max n 1) in
      List.iteri
        (fun i it ->
          let s = CArray.get arr i in
          let tag, bits =
            match it with
            | A_buffer p -> (0l, p)
            | A_i32 v -> (1l, Unsigned.UInt64.of_int64 (Int64.logand (Int64.of_int32 v) 0xFFFFFFFFL))
            | A_i64 v -> (2l, Unsigned.UInt64.of_int64 v)
            | A_f32 v -> (3l, Unsigned.UInt64.of_int64 (Int64.logand (Int64.of_int32 (Int32.bits_of_float v)) 0xFFFFFFFFL))
            | A_f64 v -> (4l, Unsigned.UInt64.of_int64 (Int64.bits_of_float v))
          in
          setf s B.arg_tag tag ;
          setf s B.arg_value bits ;
          CArray.set arr i s)
        items ;
      let dims3 (d : Framework_sig.dims) =
        CArray.of_list uint32_t (List.map Unsigned.UInt32.of_int [d.x; d.y; d.z])
      in
      let g = dims3 grid and b = dims3 block in
      let st = match stream with Some s -> s.handle | None -> Unsigned.UInt64.zero in
      let buffers = List.filter_map (function A_buffer p -> Some p | _ -> None) items in
      let from_host =
        Lazy.force Deferred.enabled
        && List.exists (fun p -> Hashtbl.mem Deferred.uploads (Deferred.key p) || Hashtbl.mem Deferred.host_copy (Deferred.key p)) buffers
      in
      (* whatever this kernel writes makes host copies that arrived earlier out of date *)
      List.iter (fun p -> Hashtbl.remove Deferred.results (Deferred.key p)) buffers ;
      if not from_host then
        B.check "sb200_kernel_launch"
          (Lazy.force B.sb200_kernel_launch k.handle (CArray.start arr) n (CArray.start g) (CArray.start b)
             (Unsigned.UInt32.of_int shared_mem) st)
      else begin
        let host_in = CArray.make (ptr void) ~initial:null (max n 1) in
        let host_out = CArray.make (ptr void) ~initial:null (max n 1) in
        let coming = CArray.make int32_t ~initial:0l (max n 1) in
        let kept = ref [] in
        List.iteri
          (fun i it ->
            match it with
            | A_buffer p ->
                (match Hashtbl.find_opt Deferred.uploads (Deferred.key p) with
                | Some (_, u) ->
                    CArray.set host_in i u.Deferred.host ;
                    kept := u.Deferred.keep :: !kept ;
                    Hashtbl.remove Deferred.uploads (Deferred.key p)
                | None -> ()) ;
                Option.iter (CArray.set host_out i) (Hashtbl.find_opt Deferred.host_copy (Deferred.key p))
            | _ -> ())
          items ;
        B.check "sb200_kernel_launch_from_host"
          (Lazy.force B.sb200_kernel_launch_from_host k.handle (CArray.start arr) n (CArray.start host_in)
             (CArray.start host_out) (CArray.start coming) (CArray.start g) (CArray.start b)
             (Unsigned.UInt32.of_int shared_mem) st) ;
        ignore (Sys.opaque_identity !kept) ;  (* the Bigarrays outlive the call, which returns after its uploads *)
        List.iteri
          (fun i it ->
            match it with
            | A_buffer p when CArray.get coming i <> 0l ->
                Hashtbl.replace Deferred.results (Deferred.key p)
                  (k.dev, raw_address_of_ptr (CArray.get host_out i), false)
            | _ -> ())
          items
      end
  end

  let enable_profiling () = ignore (Lazy.force B.sb200_enable_profiling 1)
  let disable_profiling () = ignore (Lazy.force B.sb200_enable_profiling 0)
end
