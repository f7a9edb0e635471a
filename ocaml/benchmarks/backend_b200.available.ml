(* selected by dune when sarek_b200 is present, like benchmarks/backend_cuda.available.ml *)
let init () = Sarek_b200.B200_plugin.init ()
