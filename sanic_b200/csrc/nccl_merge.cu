// Multi-device split-KV decode: each device folds its slice of the key axis into one raw
// (m, l, o) accumulator per (batch, query head); the accumulators are all-gathered over
// NCCL (NVLink / NVSwitch) and every device merges them left to right in rank order with
// the derived combine, then projects. Rank order is chunk order, so this is stage 2 of
// run_carrier_split with blocks = number of devices (reference src/interp.rs:597-640).
//
// NCCL is resolved at run time from the library already loaded in the process (the one
// torch ships) so the single-device library has no link-time dependency on it.
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <thread>

#include "common.cuh"

namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(void**, int, nccl_uid, int);
typedef int (*fn_destroy)(void*);
typedef int (*fn_allgather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef const char* (*fn_errstr)(int);
typedef int (*fn_async_err)(void*, int*);
typedef int (*fn_abort)(void*);

struct NcclApi {
    void* lib = nullptr;
    fn_get_uid get_uid = nullptr;
    fn_init_rank init_rank = nullptr;
    fn_destroy destroy = nullptr;
    fn_allgather allgather = nullptr;
    fn_errstr errstr = nullptr;
    fn_async_err async_err = nullptr;
    fn_abort abort = nullptr;
};
NcclApi g_api;

bool load_api() {
    if (g_api.lib) return true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return false;
    g_api.get_uid = (fn_get_uid)dlsym(h, "ncclGetUniqueId");
    g_api.init_rank = (fn_init_rank)dlsym(h, "ncclCommInitRank");
    g_api.destroy = (fn_destroy)dlsym(h, "ncclCommDestroy");
    g_api.allgather = (fn_allgather)dlsym(h, "ncclAllGather");
    g_api.errstr = (fn_errstr)dlsym(h, "ncclGetErrorString");
    g_api.async_err = (fn_async_err)dlsym(h, "ncclCommGetAsyncError");
    g_api.abort = (fn_abort)dlsym(h, "ncclCommAbort");
    if (!g_api.get_uid || !g_api.init_rank || !g_api.destroy || !g_api.allgather) return false;
    g_api.lib = h;
    return true;
}
constexpr int NCCL_FLOAT32 = 7;  // ncclFloat32 in nccl.h's ncclDataType_t
}  // namespace

extern "C" {

int32_t sanic_nccl_unique_id(uint8_t out_id[128]) {
    if (!out_id) return SANIC_ERR_INVALID;
    if (!load_api()) return SANIC_ERR_NCCL;
    nccl_uid id;
    if (g_api.get_uid(&id) != 0) return SANIC_ERR_NCCL;
    std::memcpy(out_id, id.internal, 128);
    return SANIC_OK;
}

int32_t sanic_nccl_init(sanic_ctx* ctx, int32_t rank, int32_t nranks, const uint8_t id[128]) {
    if (!ctx || !id) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, nranks >= 1 && rank >= 0 && rank < nranks, "nccl_init: bad rank");
    if (!load_api()) return sanic_fail(ctx, SANIC_ERR_NCCL, "nccl_init: libnccl.so.2 not found in the process");
    sanic_set_device(ctx);
    nccl_uid uid;
    std::memcpy(uid.internal, id, 128);
    void* comm = nullptr;
    int rc = g_api.init_rank(&comm, nranks, uid, rank);
    if (rc != 0)
        return sanic_fail(ctx, SANIC_ERR_NCCL, std::string("ncclCommInitRank: ") + (g_api.errstr ? g_api.errstr(rc) : "error"));
    ctx->nccl_comm = comm;
    ctx->nccl_rank = rank;
    ctx->nccl_nranks = nranks;
    return SANIC_OK;
}

int32_t sanic_nccl_shutdown(sanic_ctx* ctx) {
    if (!ctx) return SANIC_ERR_INVALID;
    if (ctx->nccl_comm && g_api.destroy) {
        sanic_set_device(ctx);
        g_api.destroy(ctx->nccl_comm);
    }
    ctx->nccl_comm = nullptr;
    ctx->nccl_nranks = 1;
    ctx->nccl_rank = 0;
    return SANIC_OK;
}

// Host-side bounded wait for the work on `stream` when it includes a collective: polls the stream and the communicator's
// asynchronous error state. A collective that a rank never joined does not complete and cannot be waited out on the
// device; when `timeout_ms` passes with the stream still busy, or the communicator reports an error, the communicator is
// aborted (its kernels stop), the context's communicator is dropped, and the call fails. With no communicator this is
// sanic_sync.
int32_t sanic_nccl_wait(sanic_ctx* ctx, void* stream, int32_t timeout_ms) {
    if (!ctx) return SANIC_ERR_INVALID;
    if (!ctx->nccl_comm || timeout_ms <= 0) return sanic_sync(ctx, stream);
    sanic_set_device(ctx);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
        if (q == cudaSuccess) return sanic_sync(ctx, stream);
        if (q != cudaErrorNotReady) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("nccl_wait: ") + cudaGetErrorString(q));
        int async = 0;
        const int rc = g_api.async_err ? g_api.async_err(ctx->nccl_comm, &async) : 0;
        const bool failed = rc != 0 || (async != 0 && async != 7 /* ncclInProgress */);
        const bool late = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > timeout_ms;
        if (failed || late) {
            if (g_api.abort) g_api.abort(ctx->nccl_comm);
            ctx->nccl_comm = nullptr; ctx->nccl_nranks = 1; ctx->nccl_rank = 0;
            return failed ? sanic_fail(ctx, SANIC_ERR_NCCL, std::string("nccl_wait: the communicator reported ") +
                                                             (g_api.errstr ? g_api.errstr(rc != 0 ? rc : async) : "an error") + "; aborted")
                          : sanic_fail(ctx, SANIC_ERR_TIMEOUT, "nccl_wait: the collective did not complete within " + std::to_string(timeout_ms) +
                                                                " ms (a rank did not take part); the communicator was aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int32_t sanic_splitkv_decode_step(sanic_ctx* ctx, const sanic_decode_params* p, float* gathered, void* out,
                                  int32_t out_dtype, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->carrier_out && gathered && out, "splitkv_decode_step: carrier_out, gathered and out are required");
    sanic_decode_params local = *p;
    const int nranks_now = ctx->nccl_comm ? ctx->nccl_nranks : 1;
    if (nranks_now == 1) {   // one device: the fold's own last-arriver merge projects straight into `out` (one launch)
        local.out = out;
        local.out_dtype = out_dtype;
        return sanic_attn_decode_splitkv(ctx, &local, stream);
    }
    local.out = nullptr;  // the local projection is meaningless before the cross-device merge
    int32_t rc = sanic_attn_decode_splitkv(ctx, &local, stream);
    if (rc != SANIC_OK) return rc;
    const int rows = p->batch * p->q_heads;
    const size_t count = (size_t)rows * (p->head_dim + 2);
    int nranks = ctx->nccl_comm ? ctx->nccl_nranks : 1;
    const float* parts = p->carrier_out;
    if (nranks > 1) {
        int nrc = g_api.allgather(p->carrier_out, gathered, count, NCCL_FLOAT32, ctx->nccl_comm, (cudaStream_t)stream);
        if (nrc != 0)
            return sanic_fail(ctx, SANIC_ERR_NCCL, std::string("ncclAllGather: ") + (g_api.errstr ? g_api.errstr(nrc) : "error"));
        parts = gathered;
    }
    return sanic_carrier_merge(ctx, parts, nranks, rows, p->head_dim, nullptr, out, out_dtype, stream);
}

}  // extern "C"
