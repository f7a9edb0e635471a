(** B200_ir_ser - Sarek IR -> S-expression text.

    The text is the "source language" of the B200 backend: [generate_source]
    returns it and [run_source] hands it to [sb200_kernel_compile], which parses
    it and recognises the kernel. One form per constructor of
    [Sarek_ir_types] (spoc/ir/Sarek_ir_types.ml); the grammar is the one in
    spoc_b200/csrc/ir.hpp of the library. *)

open Sarek_ir_types

let atom s =
  (* quote anything the reader would split *)
  let plain =
    s <> ""
    && String.for_all
         (fun c -> not (c = ' ' || c = '(' || c = ')' || c = '"' || c = ';' || c = '\n' || c = '\t'))
         s
  in
  if plain then s else "\"" ^ String.escaped s ^ "\""

let list items = "(" ^ String.concat " " items ^ ")"

let memspace = function Global -> "global" | Shared -> "shared" | Local -> "local"

let rec elt = function
  | TInt32 -> "i32"
  | TInt64 -> "i64"
  | TFloat32 -> "f32"
  | TFloat64 -> "f64"
  | TBool -> "bool"
  | TUnit -> "unit"
  | TRecord (n, _) -> list ["record"; atom n]
  | TVariant (n, _) -> list ["variant"; atom n]
  | TArray (t, m) -> list ["array"; elt t; memspace m]
  | TVec t -> list ["vecof"; elt t]

let const = function
  | CInt32 n -> list ["const"; "i32"; Int32.to_string n]
  | CInt64 n -> list ["const"; "i64"; Int64.to_string n]
  | CFloat32 f -> list ["const"; "f32"; Printf.sprintf "%.17g" f]
  | CFloat64 f -> list ["const"; "f64"; Printf.sprintf "%.17g" f]
  | CBool b -> list ["const"; "bool"; string_of_bool b]
  | CUnit -> list ["const"; "unit"; "0"]

let binop = function
  | Add -> "add" | Sub -> "sub" | Mul -> "mul" | Div -> "div" | Mod -> "mod"
  | Eq -> "eq" | Ne -> "ne" | Lt -> "lt" | Le -> "le" | Gt -> "gt" | Ge -> "ge"
  | And -> "and" | Or -> "or" | Shl -> "shl" | Shr -> "shr"
  | BitAnd -> "band" | BitOr -> "bor" | BitXor -> "bxor"

let unop = function Neg -> "neg" | Not -> "not" | BitNot -> "bnot"

let evar (v : var) = list ["evar"; atom v.var_name; string_of_int v.var_id]

let rec expr = function
  | EConst c -> const c
  | EVar v -> evar v
  | EBinop (op, a, b) -> list ["binop"; binop op; expr a; expr b]
  | EUnop (op, a) -> list ["unop"; unop op; expr a]
  | EArrayRead (arr, idx) -> list ["read"; atom arr; expr idx]
  | EArrayReadExpr (base, idx) -> list ["readexpr"; expr base; expr idx]
  | ERecordField (e, f) -> list ["field"; expr e; atom f]
  | EIntrinsic (path, name, args) ->
      list (["intrinsic"; list (List.map atom path); atom name] @ List.map expr args)
  | ECast (t, e) -> list ["cast"; elt t; expr e]
  | ETuple es -> list ("tuple" :: List.map expr es)
  | EApp (f, args) -> list ("app" :: expr f :: List.map expr args)
  | ERecord (n, fields) ->
      list ("mkrecord" :: atom n :: List.map (fun (f, e) -> list [atom f; expr e]) fields)
  | EVariant (t, c, args) -> list ("mkvariant" :: atom t :: atom c :: List.map expr args)
  | EArrayLen arr -> list ["arraylen"; atom arr]
  | EArrayCreate (t, size, m) -> list ["arraycreate"; elt t; expr size; memspace m]
  | EIf (c, a, b) -> list ["if"; expr c; expr a; expr b]
  | EMatch (e, _) -> list ["match"; expr e]

let rec lvalue = function
  | LVar v -> list ["lvar"; atom v.var_name; string_of_int v.var_id]
  | LArrayElem (arr, idx) -> list ["elem"; atom arr; expr idx]
  | LArrayElemExpr (base, idx) -> list ["elemexpr"; expr base; expr idx]
  | LRecordField (lv, f) -> list ["lfield"; lvalue lv; atom f]

let rec stmt = function
  | SAssign (lv, e) -> list ["assign"; lvalue lv; expr e]
  | SSeq ss -> list ("seq" :: List.map stmt ss)
  | SIf (c, a, None) -> list ["sif"; expr c; stmt a]
  | SIf (c, a, Some b) -> list ["sif"; expr c; stmt a; stmt b]
  | SWhile (c, b) -> list ["while"; expr c; stmt b]
  | SFor (v, lo, hi, dir, b) ->
      list
        [ "for"; atom v.var_name; string_of_int v.var_id; expr lo; expr hi;
          (match dir with Upto -> "upto" | Downto -> "downto"); stmt b ]
  | SMatch (e, _) -> list ["match"; expr e]
  | SReturn e -> list ["return"; expr e]
  | SBarrier -> "(barrier)"
  | SWarpBarrier -> "(warpbarrier)"
  | SExpr e -> list ["expr"; expr e]
  | SEmpty -> "(empty)"
  | SLet (v, e, b) ->
      list ["let"; atom v.var_name; string_of_int v.var_id; elt v.var_type; expr e; stmt b]
  | SLetMut (v, e, b) ->
      list ["letmut"; atom v.var_name; string_of_int v.var_id; elt v.var_type; expr e; stmt b]
  | SPragma (hints, b) -> list ["pragma"; list (List.map atom hints); stmt b]
  | SMemFence -> "(memfence)"
  | SBlock b -> list ["block"; stmt b]
  | SNative _ -> "(native)"

let param = function
  | DParam (v, Some info) ->
      Some (list ["vec"; atom v.var_name; string_of_int v.var_id; elt info.arr_elttype])
  | DParam (v, None) ->
      Some (list ["scalar"; atom v.var_name; string_of_int v.var_id; elt v.var_type])
  | DLocal _ | DShared _ -> None

(** The whole kernel. Constructs the backend does not run ([match], [native],
    records, helper functions) are printed as opaque forms, which the library
    answers with Unsupported_construct. *)
let to_sexp (k : kernel) : string =
  list
    [ "kernel"; atom k.kern_name;
      list ("params" :: List.filter_map param k.kern_params);
      list ["body"; stmt k.kern_body] ]
