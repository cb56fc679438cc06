// Entry points still to be written; each reports HB_ERR_UNSUPPORTED.
#include "hb_internal.h"
#define STUB(ctx, name) return hb_fail(ctx, HB_ERR_UNSUPPORTED, name ": not built yet")
extern "C" hb_status hb_rmsnorm(hb_ctx* ctx, const void*, const void*, void*, void*, int64_t, int64_t, float) { STUB(ctx, "rmsnorm"); }
extern "C" hb_status hb_rope(hb_ctx* ctx, void*, int64_t, int64_t, int64_t, int64_t, int64_t, float, int64_t) { STUB(ctx, "rope"); }
extern "C" hb_status hb_embedding(hb_ctx* ctx, const void*, const int32_t*, void*, int64_t, int64_t, int64_t) { STUB(ctx, "embedding"); }
extern "C" hb_status hb_swiglu(hb_ctx* ctx, const void*, void*, int64_t, int64_t) { STUB(ctx, "swiglu"); }
extern "C" hb_status hb_gelu(hb_ctx* ctx, const void*, void*, int64_t) { STUB(ctx, "gelu"); }
extern "C" hb_status hb_add(hb_ctx* ctx, const void*, const void*, void*, int64_t) { STUB(ctx, "add"); }
extern "C" hb_status hb_argmax(hb_ctx* ctx, const void*, int32_t*, int64_t, int64_t) { STUB(ctx, "argmax"); }
extern "C" hb_status hb_comm_unique_id(void*) { return HB_ERR_UNSUPPORTED; }
extern "C" hb_status hb_comm_init_rank(hb_ctx* ctx, int32_t, int32_t, const void*) { STUB(ctx, "comm_init_rank"); }
extern "C" hb_status hb_comm_destroy(hb_ctx*) { return HB_OK; }
extern "C" hb_status hb_p2p_alloc(hb_ctx* ctx, size_t, void**, void*) { STUB(ctx, "p2p_alloc"); }
extern "C" hb_status hb_p2p_attach(hb_ctx* ctx, int32_t, int32_t, const void*, size_t) { STUB(ctx, "p2p_attach"); }
extern "C" hb_status hb_all_reduce(hb_ctx* ctx, void*, int64_t, int32_t, int32_t) { STUB(ctx, "all_reduce"); }
