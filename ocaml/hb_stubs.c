/* UNCOMPILED / UNVERIFIED: C stubs between OCaml `external`s (model_ir.ml) and the C ABI
 * of libhabu_b200.so.  Each stub unpacks OCaml values into plain pointers and sizes and
 * forwards; only hb_sync releases the runtime lock, because every other entry point is
 * asynchronous and returns at once. */
#include <caml/alloc.h>
#include <caml/bigarray.h>
#include <caml/custom.h>
#include <caml/memory.h>
#include <caml/mlvalues.h>
#include <caml/threads.h>
#include <string.h>

#include "habu_b200.h"

#define Ctx_val(v) (*((hb_ctx**)Data_custom_val(v)))
#define Buf_val(v) (*((void**)Data_custom_val(v)))

static void ctx_finalize(value v) { if (Ctx_val(v)) hb_ctx_destroy(Ctx_val(v)); }
static struct custom_operations ctx_ops = {"habu_b200.ctx", ctx_finalize, custom_compare_default, custom_hash_default,
                                           custom_serialize_default, custom_deserialize_default,
                                           custom_compare_ext_default, custom_fixed_length_default};
static struct custom_operations buf_ops = {"habu_b200.buffer", custom_finalize_default, custom_compare_default,
                                           custom_hash_default, custom_serialize_default, custom_deserialize_default,
                                           custom_compare_ext_default, custom_fixed_length_default};

static value make_result(int ok, value payload) {   /* Ok payload | Error payload */
  CAMLparam1(payload);
  CAMLlocal1(r);
  r = caml_alloc(1, ok ? 0 : 1);
  Store_field(r, 0, payload);
  CAMLreturn(r);
}

/* { buf; offset; dtype; shape; stride } -> hb_tensor */
static hb_tensor tensor_of_value(value t) {
  hb_tensor o;
  memset(&o, 0, sizeof(o));
  int dtype = Int_val(Field(t, 2));
  size_t es = dtype == HB_BF16 ? 2 : 4;
  o.ptr = (char*)Buf_val(Field(t, 0)) + (size_t)Long_val(Field(t, 1)) * es;
  o.dtype = dtype;
  o.rank = (int32_t)Wosize_val(Field(t, 3));
  for (int i = 0; i < o.rank && i < 4; ++i) {
    o.shape[i] = Long_val(Field(Field(t, 3), i));
    o.stride[i] = Long_val(Field(Field(t, 4), i));
  }
  return o;
}

CAMLprim value caml_hb_ctx_create(value device) {
  CAMLparam1(device);
  CAMLlocal1(v);
  hb_ctx* c = NULL;
  hb_status st = hb_ctx_create(Int_val(device), &c);
  if (st != HB_OK) CAMLreturn(make_result(0, Val_int(st)));
  v = caml_alloc_custom(&ctx_ops, sizeof(hb_ctx*), 0, 1);
  Ctx_val(v) = c;
  CAMLreturn(make_result(1, v));
}

CAMLprim value caml_hb_last_error_string(value ctx) { return caml_copy_string(hb_last_error_string(Ctx_val(ctx))); }

CAMLprim value caml_hb_alloc(value ctx, value bytes) {
  CAMLparam2(ctx, bytes);
  CAMLlocal1(v);
  void* p = NULL;
  hb_status st = hb_alloc(Ctx_val(ctx), (size_t)Long_val(bytes), &p);
  if (st != HB_OK) CAMLreturn(make_result(0, Val_int(st)));
  v = caml_alloc_custom(&buf_ops, sizeof(void*), 0, 1);
  Buf_val(v) = p;
  CAMLreturn(make_result(1, v));
}

CAMLprim value caml_hb_upload(value ctx, value buf, value ba) {
  return Val_int(hb_upload(Ctx_val(ctx), Buf_val(buf), Caml_ba_data_val(ba), caml_ba_byte_size(Caml_ba_array_val(ba))));
}
CAMLprim value caml_hb_download(value ctx, value ba, value buf) {
  return Val_int(hb_download(Ctx_val(ctx), Caml_ba_data_val(ba), Buf_val(buf), caml_ba_byte_size(Caml_ba_array_val(ba))));
}
CAMLprim value caml_hb_sync(value ctx) {
  hb_ctx* c = Ctx_val(ctx);
  caml_release_runtime_system();
  hb_status st = hb_sync(c);
  caml_acquire_runtime_system();
  return Val_int(st);
}

CAMLprim value caml_hb_matmul(value ctx, value a, value b, value out, value epi, value residual) {
  hb_tensor ta = tensor_of_value(a), tb = tensor_of_value(b), tc = tensor_of_value(out);
  hb_matmul_opts o = {Int_val(epi), -1, NULL, 0};
  if (Is_block(residual)) {
    hb_tensor r = tensor_of_value(Field(residual, 0));
    o.residual = r.ptr;
    o.residual_ld = r.stride[0];
  }
  return Val_int(hb_matmul(Ctx_val(ctx), &ta, &tb, &tc, &o));
}
CAMLprim value caml_hb_matmul_bytecode(value* argv, int argn) {
  (void)argn;
  return caml_hb_matmul(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5]);
}

CAMLprim value caml_hb_attention(value ctx, value q, value k, value v, value out, value causal, value scale) {
  hb_tensor tq = tensor_of_value(q), tk = tensor_of_value(k), tv = tensor_of_value(v), to = tensor_of_value(out);
  hb_attn_opts o = {Bool_val(causal), (float)Double_val(scale), NULL, -1};
  return Val_int(hb_attention(Ctx_val(ctx), &tq, &tk, &tv, &to, &o));
}
CAMLprim value caml_hb_attention_bytecode(value* argv, int argn) {
  (void)argn;
  return caml_hb_attention(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6]);
}

CAMLprim value caml_hb_all_reduce(value ctx, value x, value algo) {
  hb_tensor t = tensor_of_value(x);
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.shape[i];
  return Val_int(hb_all_reduce(Ctx_val(ctx), t.ptr, n, t.dtype, Int_val(algo)));
}

CAMLprim value caml_hb_autotune(value ctx, value m, value n, value k, value layout, value epi) {
  /* CAMLparam takes at most five values; the sixth is registered with CAMLxparam */
  CAMLparam5(ctx, m, n, k, layout);
  CAMLxparam1(epi);
  CAMLlocal2(pair, ms);
  hb_op_desc d = {HB_OP_MATMUL, HB_BF16, Long_val(m), Long_val(n), Long_val(k), Int_val(layout), Int_val(epi)};
  hb_tune_result r;
  hb_status st = hb_autotune(Ctx_val(ctx), &d, HB_TUNE_SEARCH, &r);
  /* allocate the float first, into a registered local: an allocation inside the argument of
   * Store_field could move `pair` after its field address had been computed */
  ms = caml_copy_double(st == HB_OK ? r.ms : 0.0);
  pair = caml_alloc_tuple(2);
  Store_field(pair, 0, Val_int(st == HB_OK ? r.config_id : -st));
  Store_field(pair, 1, ms);
  CAMLreturn(pair);
}
CAMLprim value caml_hb_autotune_bytecode(value* argv, int argn) {
  (void)argn;
  return caml_hb_autotune(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5]);
}
