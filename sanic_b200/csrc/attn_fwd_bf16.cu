#include "common.cuh"
extern "C" int32_t sanic_attn_fwd_bf16(sanic_ctx* ctx, const sanic_attn_params* p, void* stream) {
    (void)p; (void)stream;
    return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "attn_fwd_bf16: not built yet");
}
