// Split-KV decode: the online-softmax fold over a KV cache for one query token per
// sequence, as a two-stage split reduction (reference src/interp.rs:555-643).
//
// Stage 1 (this kernel's main loop): CTA (split, kv head, batch) streams its contiguous
// chunk of the key axis through shared memory (16-byte cp.async, multi-stage ring) and
// folds it on the tensor cores: the GQA group's query heads are the rows of a 16-row
// A operand, S = Q K^T and O += P V are m16n8k16 bf16 MMAs with f32 accumulators, the
// (m, l, o) carrier stays in registers. Each of the 4 warps owns 16 keys of every
// 64-key tile and keeps its own carrier; warps are merged once at the end with the
// carrier's combine.
// Stage 2: the last CTA to finish a (batch, kv head) merges the per-chunk partials left
// to right with the derived combine (-inf guard included, src/derive.rs:1700-1713) and
// projects o / l, or exports the merged raw accumulator for a cross-device merge.
//
// HBM-bound: algorithmic bytes = 2 * kv_len * D * 2 per (batch, kv head).
#include <atomic>

#include "common.cuh"

#include "attn_decode_body.cuh"

namespace {
using namespace sanic;
using namespace sanic::decode;

template <int D, bool VT, bool SPLITP>
__global__ void __launch_bounds__(128) attn_decode_kernel(sanic_decode_params p, int* counters, int* err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    attn_decode_tile<D, VT, SPLITP>(p, counters, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, smem_raw, (int)threadIdx.x, true, 0, err);
}

// Stage 2 on its own: merge n_parts raw accumulators and project.
__global__ void carrier_merge_kernel(const float* parts, int n_parts, int rows, int D, float* carrier_out, void* out,
                                     int out_dtype) {
    int row = blockIdx.x;
    const int W = D + 2;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float* pa = parts + (size_t)row * W;
        float m = pa[0], l = pa[1], ov = pa[2 + d];
        for (int s = 1; s < n_parts; ++s) {
            const float* pb = parts + ((size_t)s * rows + row) * W;
            MloScale sc = mlo_rescale(m, pb[0]);
            l = l * sc.ra + pb[1] * sc.rb; ov = ov * sc.ra + pb[2 + d] * sc.rb; m = sc.m;
        }
        if (carrier_out) {
            float* c = carrier_out + (size_t)row * W;
            c[2 + d] = ov;
            if (d == 0) { c[0] = m; c[1] = l; }
        }
        if (out) {
            float v = ov / l;
            if (out_dtype == SANIC_BF16) ((uint16_t*)out)[(size_t)row * D + d] = f32_to_bf16_bits(v);
            else ((float*)out)[(size_t)row * D + d] = v;
        }
    }
}

template <int D, bool VT>
int32_t launch_decode(sanic_ctx* ctx, const sanic_decode_params& p, cudaStream_t st) {
    // SANIC_DECODE_SPLIT_P=1: the bf16 remainder of P goes through a second MMA (error measurements, A/B timing)
    static const bool split_p = getenv("SANIC_DECODE_SPLIT_P") && getenv("SANIC_DECODE_SPLIT_P")[0] == '1';
    auto kern = split_p ? attn_decode_kernel<D, VT, true> : attn_decode_kernel<D, VT, false>;
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM));
    int* counters = (int*)(p.partials + (size_t)p.batch * p.q_heads * p.n_splits * (D + 2));
    dim3 grid(p.n_splits, p.kv_heads, p.batch);
    cudaError_t le = launch_pdl(kern, grid, dim3(128), (size_t)Cfg<D>::SMEM, st, p, counters, ctx->status_dev);
    if (le != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("attn_decode_splitkv: ") + cudaGetErrorString(le));
    return SANIC_OK;
}
}  // namespace

extern "C" {

// partials [B*Hq, n_splits, 2+D] floats followed by one int32 ticket counter per
// (batch, kv head); kv heads <= q heads bounds the counter block.
size_t sanic_attn_decode_scratch_bytes(int32_t batch, int32_t q_heads, int32_t head_dim, int32_t n_splits) {
    return ((size_t)batch * q_heads * n_splits * (head_dim + 2) + (size_t)batch * q_heads) * 4;
}

int32_t sanic_attn_decode_suggest_splits(sanic_ctx* ctx, int32_t batch, int32_t kv_heads, int32_t head_dim, int64_t kv_len) {
    if (!ctx || batch <= 0 || kv_heads <= 0) return 1;
    int64_t tiles = (kv_len + KT - 1) / KT;
    if (tiles < 1) tiles = 1;
    int per_sm = (head_dim == 128) ? 2 : 4;       // resident CTAs per SM by shared memory
    int64_t waves = 4;                            // a few waves hide the tail
    int64_t target = (int64_t)ctx->sm_count * per_sm * waves / ((int64_t)batch * kv_heads);
    if (target < 1) target = 1;
    // keep at least 4 tiles per chunk so the cp.async ring fills
    int64_t cap = tiles / 4 > 0 ? tiles / 4 : 1;
    if (target > cap) target = cap;
    if (target > 4096) target = 4096;
    return (int32_t)target;
}

static int32_t decode_validate_and_launch(sanic_ctx* ctx, const sanic_decode_params* p, void* stream);

int32_t sanic_attn_decode_splitkv(sanic_ctx* ctx, const sanic_decode_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    return decode_validate_and_launch(ctx, p, stream);
}

// ── the entry point for callers that cannot allocate ──
// Scratch for the split-KV fold lives in this file-scope device array instead of a buffer the
// caller allocates. Every device that loads the library holds these bytes until the process exits.
#define SANIC_STATIC_SCRATCH_FLOATS (1u << 20)   /* 4 MiB of partial accumulators */
#define SANIC_STATIC_SCRATCH_COUNTERS 4096u      /* one ticket per (batch, kv head) */
static __device__ __align__(256) float g_decode_scratch[SANIC_STATIC_SCRATCH_FLOATS + SANIC_STATIC_SCRATCH_COUNTERS];

size_t sanic_attn_decode_static_scratch_capacity(void) { return (size_t)SANIC_STATIC_SCRATCH_FLOATS * sizeof(float); }

int32_t sanic_attn_decode_splitkv_static(sanic_ctx* ctx, const sanic_decode_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->batch > 0 && p->q_heads > 0 && p->kv_heads > 0 && p->n_splits >= 1 && p->head_dim > 0,
                  "attn_decode_static: bad shape");
    const size_t need = (size_t)p->batch * p->q_heads * p->n_splits * (p->head_dim + 2);
    if (need > SANIC_STATIC_SCRATCH_FLOATS)
        return sanic_fail(ctx, SANIC_ERR_INVALID,
                          "attn_decode_static: batch*q_heads*n_splits*(head_dim+2) = " + std::to_string(need) +
                          " floats exceeds the built-in scratch of " + std::to_string(SANIC_STATIC_SCRATCH_FLOATS) +
                          " floats; use fewer splits or sanic_attn_decode_splitkv with caller scratch");
    if ((size_t)p->batch * p->kv_heads > SANIC_STATIC_SCRATCH_COUNTERS)
        return sanic_fail(ctx, SANIC_ERR_INVALID,
                          "attn_decode_static: batch*kv_heads = " + std::to_string((size_t)p->batch * p->kv_heads) +
                          " exceeds the built-in " + std::to_string(SANIC_STATIC_SCRATCH_COUNTERS) +
                          " ticket counters; use sanic_attn_decode_splitkv with caller scratch");
    sanic_set_device(ctx);
    // In host code the array's name is only a handle. Its device address is looked up once per
    // device, with that device current; the kernel is given that address, never the name.
    // Two host threads may both find the slot empty and both look the address up: they store the
    // same value, so the slots are atomics only to make that overlap well defined.
    static std::atomic<float*> dev_addr[64];
    SANIC_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "attn_decode_static: device ordinal out of range");
    float* scratch = dev_addr[ctx->device].load(std::memory_order_acquire);
    if (!scratch) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
        if (e != cudaSuccess || !ptr)
            return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("attn_decode_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        scratch = (float*)ptr;
        dev_addr[ctx->device].store(scratch, std::memory_order_release);
    }
    sanic_decode_params local = *p;
    local.partials = scratch;
    // an invalid call must not touch the shared array: validate first, then clear the counters
    int32_t rc = host_validate(ctx, &local);
    if (rc != SANIC_OK) return rc;
    // The ticket counters must start at zero. They sit right after this call's partials; the array
    // keeps whatever the previous call left, so clear them on the stream (no allocation involved).
    SANIC_CUDA_CHECK(ctx, cudaMemsetAsync(scratch + need, 0, (size_t)p->batch * p->kv_heads * sizeof(int), (cudaStream_t)stream));
    return decode_validate_and_launch(ctx, &local, stream);
}

static int32_t decode_validate_and_launch(sanic_ctx* ctx, const sanic_decode_params* p, void* stream) {
    int32_t rc = host_validate(ctx, p);
    if (rc != SANIC_OK) return rc;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (p->head_dim == 128) return p->v_transposed ? launch_decode<128, true>(ctx, *p, st) : launch_decode<128, false>(ctx, *p, st);
    return p->v_transposed ? launch_decode<64, true>(ctx, *p, st) : launch_decode<64, false>(ctx, *p, st);
}

int32_t sanic_carrier_merge(sanic_ctx* ctx, const float* parts, int32_t n_parts, int32_t rows, int32_t head_dim,
                            float* carrier_out, void* out, int32_t out_dtype, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, parts && n_parts >= 1 && rows >= 1 && head_dim >= 1, "carrier_merge: bad arguments");
    SANIC_REQUIRE(ctx, out || carrier_out, "carrier_merge: no output requested");
    sanic_set_device(ctx);
    carrier_merge_kernel<<<rows, 128, 0, (cudaStream_t)stream>>>(parts, n_parts, rows, head_dim, carrier_out, out, out_dtype);
    SANIC_LAUNCH_CHECK(ctx, "carrier_merge");
    return SANIC_OK;
}

}  // extern "C"
