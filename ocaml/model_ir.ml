(* UNCOMPILED / UNVERIFIED source: the build image has no OCaml toolchain.

   Model-IR operator nodes over libhabu_b200.so.  Conventions follow the reference:
   errors are values over polymorphic variants (src/lib/error.ml:18-26), constructors
   validate and return a result (src/lib/sleigh.ml:50-62), records derive sexp. *)
open Sexplib.Std

type error =
  [ `Invalid of string | `Not_found of string | `Duplicate of string
  | `Cuda of string | `Nccl of string | `Timeout of string
  | `Unsupported of string | `No_memory of string ]
[@@deriving sexp]

type dtype = F32 | Bf16 | I32 [@@deriving sexp]
type ctx                                   (* hb_ctx*, custom block with finaliser *)
type buffer                                (* device pointer owned by a ctx *)

type tensor = { buf : buffer; offset : int; dtype : dtype; shape : int array; stride : int array }

module Epilogue = struct
  type t = None_ | Gelu | Swiglu | Residual of tensor
end

external ctx_create : int -> (ctx, int) result = "caml_hb_ctx_create"
external last_error : ctx -> string = "caml_hb_last_error_string"
external alloc : ctx -> int -> (buffer, int) result = "caml_hb_alloc"
external upload : ctx -> buffer -> ('a, 'b, Bigarray.c_layout) Bigarray.Genarray.t -> int = "caml_hb_upload"
external download : ctx -> ('a, 'b, Bigarray.c_layout) Bigarray.Genarray.t -> buffer -> int = "caml_hb_download"
(* the only call that blocks; the stub releases the runtime lock around it *)
external sync : ctx -> int = "caml_hb_sync"
external matmul_raw : ctx -> tensor -> tensor -> tensor -> int -> tensor option -> int = "caml_hb_matmul_bytecode" "caml_hb_matmul"
external attention_raw : ctx -> tensor -> tensor -> tensor -> tensor -> bool -> float -> int = "caml_hb_attention_bytecode" "caml_hb_attention"
external all_reduce_raw : ctx -> tensor -> int -> int = "caml_hb_all_reduce"
external autotune_raw : ctx -> int -> int -> int -> int -> int -> int * float = "caml_hb_autotune_bytecode" "caml_hb_autotune"

let to_error ctx = function
  | 1 -> `Invalid (last_error ctx) | 2 -> `Not_found (last_error ctx) | 3 -> `Duplicate (last_error ctx)
  | 4 -> `Cuda (last_error ctx) | 5 -> `Nccl (last_error ctx) | 6 -> `Timeout (last_error ctx)
  | 7 -> `Unsupported (last_error ctx) | _ -> `No_memory (last_error ctx)

let check ctx st = if st = 0 then Ok () else Error (to_error ctx st)

(* the model-IR nodes *)
let matmul ctx ?(epilogue = Epilogue.None_) ~a ~b ~out () =
  let code, r = match epilogue with
    | Epilogue.None_ -> 0, None | Gelu -> 1, None | Swiglu -> 2, None | Residual r -> 3, Some r in
  check ctx (matmul_raw ctx a b out code r)

let attention ctx ?(causal = true) ~scale ~q ~k ~v ~out () =
  check ctx (attention_raw ctx q k v out causal scale)

let all_reduce ctx ?(algo = 0) x = check ctx (all_reduce_raw ctx x algo)

(* autotune entry point: returns (config_id, milliseconds) of the winner *)
let autotune ctx ~m ~n ~k ?(layout = 0) ?(epilogue = 0) () =
  let id, ms = autotune_raw ctx m n k layout epilogue in
  if id < 0 then Error (to_error ctx (-id)) else Ok (id, ms)
