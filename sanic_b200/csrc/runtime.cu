// Context, memory and emitter selection: the runtime half that replaces the
// reference's Metal device layer (src/metal.rs:149-490 in the reference project).
#include <cstring>
#include <new>

#include "common.cuh"

extern "C" {

const char* sanic_version(void) { return "sanic_b200 0.1 (sm_100a)"; }

int32_t sanic_cuda_open(int32_t ordinal, sanic_ctx** out) {
    if (!out) return SANIC_ERR_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return SANIC_ERR_CUDA;
    if (ordinal < 0 || ordinal >= n) return SANIC_ERR_INVALID;
    sanic_ctx* ctx = new (std::nothrow) sanic_ctx();
    if (!ctx) return SANIC_ERR_NOMEM;
    ctx->device = ordinal;
    cudaDeviceProp prop;
    if (cudaSetDevice(ordinal) != cudaSuccess || cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) {
        delete ctx;
        return SANIC_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem = (int)prop.sharedMemPerBlockOptin;
    ctx->l2_bytes = prop.l2CacheSize;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->hbm_bytes = prop.totalGlobalMem;
    if (prop.major != 10) {
        // The kernels are built for sm_100a only; there is no other code path.
        delete ctx;
        return SANIC_ERR_UNSUPPORTED;
    }
    if (cudaHostAlloc((void**)&ctx->status_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void**)&ctx->status_dev, ctx->status_host, 0) != cudaSuccess) {
        delete ctx;
        return SANIC_ERR_CUDA;
    }
    *ctx->status_host = 0;
    *out = ctx;
    return SANIC_OK;
}

int32_t sanic_cuda_close(sanic_ctx* ctx) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_nccl_shutdown(ctx);
    if (ctx->status_host) { cudaSetDevice(ctx->device); cudaFreeHost(ctx->status_host); }
    delete ctx;
    return SANIC_OK;
}

const char* sanic_last_error(sanic_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int32_t sanic_specs(sanic_ctx* ctx, sanic_device_specs* out) {
    if (!ctx || !out) return SANIC_ERR_INVALID;
    out->sm_count = ctx->sm_count;
    out->cc_major = ctx->cc_major;
    out->cc_minor = ctx->cc_minor;
    out->max_smem_per_block = ctx->max_smem;
    out->l2_bytes = ctx->l2_bytes;
    out->warp = 32;
    out->hbm_bytes = ctx->hbm_bytes;
    out->hbm_gbs_nominal = 7700.0;
    out->bf16_tflops_nominal = 2250.0;
    return SANIC_OK;
}

int32_t sanic_alloc(sanic_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaMalloc(dptr, bytes ? bytes : 1));
    return SANIC_OK;
}
int32_t sanic_free(sanic_ctx* ctx, void* dptr) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaFree(dptr));
    return SANIC_OK;
}
int32_t sanic_upload(sanic_ctx* ctx, void* dst, const void* src, size_t bytes, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return SANIC_OK;
}
int32_t sanic_download(sanic_ctx* ctx, void* dst, const void* src, size_t bytes, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SANIC_CUDA_CHECK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return SANIC_OK;
}
int32_t sanic_memset(sanic_ctx* ctx, void* dptr, int32_t byte, size_t bytes, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaMemsetAsync(dptr, byte, bytes, (cudaStream_t)stream));
    return SANIC_OK;
}
int32_t sanic_sync(sanic_ctx* ctx, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    // a kernel whose bounded wait ran out left its code in the status word
    int code = *(volatile int*)ctx->status_host;
    if (code != 0) {
        *ctx->status_host = 0;
        if (code == 51) return sanic_fail(ctx, SANIC_ERR_INVALID, "a gather index was out of range (code 51)");
        if (code == 52)
            return sanic_fail(ctx, SANIC_ERR_INVALID, "a device-side key length was outside [1, kv_cap] and was clamped: the decode "
                                                      "position ran past the cache extent (code 52)");
        return sanic_fail(ctx, SANIC_ERR_TIMEOUT, "a bounded device-side wait ran out (code " + std::to_string(code) + ")");
    }
    return SANIC_OK;
}

int32_t sanic_status_inject(sanic_ctx* ctx, int32_t code) {
    if (!ctx || !ctx->status_host) return SANIC_ERR_INVALID;
    *(volatile int*)ctx->status_host = code;
    return SANIC_OK;
}

// Kernel selection keyed on slot kinds and leaf structure only.
int32_t sanic_emit_select(const sanic_carrier_desc* c, int32_t* family) {
    if (!c || !family) return SANIC_ERR_INVALID;
    *family = SANIC_KERNEL_NONE;
    if (c->n_slots == 3 && c->kind[0] == SANIC_SLOT_PLAIN_MAX && c->kind[1] == SANIC_SLOT_EXP_SHIFTED &&
        c->kind[2] == SANIC_SLOT_EXP_SHIFTED && c->ref[1] == 0 && c->ref[2] == 0 && c->in_body_contraction) {
        *family = SANIC_KERNEL_ONLINE_SOFTMAX_FOLD;
    } else if (c->n_slots == 2 && c->kind[0] == SANIC_SLOT_PLAIN_ADD && c->kind[1] == SANIC_SLOT_PLAIN_ADD &&
               c->deferred_div) {
        *family = SANIC_KERNEL_DEFERRED_NORM_CONTRACTION;
    } else if (c->n_slots == 1 && c->kind[0] == SANIC_SLOT_PLAIN_ADD && c->leaf_dtype == SANIC_I4) {
        *family = SANIC_KERNEL_GROUPED_I4_CONTRACTION;
    } else if (c->n_slots == 1 && c->kind[0] == SANIC_SLOT_PLAIN_ADD) {
        *family = SANIC_KERNEL_PLAIN_CONTRACTION;
    } else if (c->n_slots == 2 && c->kind[0] == SANIC_SLOT_PLAIN_MAX && c->kind[1] == SANIC_SLOT_AT_EXTREMUM &&
               c->ref[1] == 0) {
        *family = SANIC_KERNEL_EXTREMUM_INDEX;
    } else {
        return SANIC_ERR_UNSUPPORTED;
    }
    return SANIC_OK;
}

}  // extern "C"
