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

// The same fold with the (batch, kv head, key tile) space cut into one contiguous range per CTA of a grid that is
// exactly resident (stream-K): every tile costs the same, so all CTAs finish together and there is no last partial wave,
// which a fixed grid of chunks pays when a device's slice is short (8 devices: 2 GB per device, four waves). A CTA's range
// crosses at most a few (batch, kv head) groups; each crossing is one segment with its own partial slot, and the group's
// last segment to arrive runs stage 2. With an exchange (several devices) stage 2 also stores the group's merged
// accumulators into every device's buffer and publishes the group's flag; the CTA finishes its own range first and only
// then waits for the other devices' flags of the groups it owes, merges them in rank order and projects: the whole
// multi-device step is this one launch.
template <int D, bool VT, bool SPLITP>
__global__ void __launch_bounds__(128) attn_decode_streamk_kernel(sanic_decode_params p, int* counters, int* err, Exchange x, int use_x) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int tid = threadIdx.x;
    griddep_launch();
    griddep_wait();
    const KeyRange kr = key_range(p, tid, err);
    const long long nT = kr.T1 - kr.T0;
    const int groups = p.batch * p.kv_heads;
    const long long T = nT * groups;
    const long long G = T < (long long)gridDim.x ? T : (long long)gridDim.x;     // every CTA below G owns at least one tile
    const long long c = blockIdx.x;
    if (c >= G) return;
    long long cur = c * T / G;
    const long long end = (c + 1) * T / G;
    auto cta_of = [&](long long tile) { return ((tile + 1) * G - 1) / T; };      // the CTA whose range holds a global tile
    constexpr int MAX_OWED = 8;
    int owed[MAX_OWED];
    int n_owed = 0;
    while (cur < end) {
        const int gi = (int)(cur / nT);
        const int t0 = (int)(cur % nT);
        const long long left = end - cur;
        const int t1 = (int)((long long)t0 + left < nT ? (long long)t0 + left : nT);
        const int b = gi / p.kv_heads, hk = gi % p.kv_heads;
        const long long c_first = cta_of((long long)gi * nT), c_last = cta_of((long long)(gi + 1) * nT - 1);
        const int slot = (int)(c - c_first), n_parts = (int)(c_last - c_first + 1);
        if (n_parts > p.n_splits || slot < 0 || slot >= n_parts) {      // the host sized the scratch for fewer segments per group
            if (tid == 0 && err) atomicCAS(err, 0, 53);
            return;
        }
        if (fold_segment<D, VT, SPLITP>(p, counters, b, hk, kr.T0 + t0, kr.T0 + t1, kr.lo, kr.hi, slot, n_parts, smem_raw, tid, 0)) {
            merge_group<D>(p, b, hk, n_parts, tid, 0, use_x ? &x : nullptr);
            if (use_x) {
                if (n_owed < MAX_OWED) owed[n_owed++] = gi;
                else if (!merge_group_remote<D>(p, b, hk, tid, 0, &x, err)) return;
            }
        }
        cur += t1 - t0;
    }
    for (int i = 0; i < n_owed; ++i)
        if (!merge_group_remote<D>(p, owed[i] / p.kv_heads, owed[i] % p.kv_heads, tid, 0, &x, err)) return;
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
template <int D, bool VT>
int32_t launch_streamk(sanic_ctx* ctx, const sanic_decode_params& p, cudaStream_t st, const Exchange* x) {
    static const bool split_p = getenv("SANIC_DECODE_SPLIT_P") && getenv("SANIC_DECODE_SPLIT_P")[0] == '1';
    auto kern = split_p ? attn_decode_streamk_kernel<D, VT, true> : attn_decode_streamk_kernel<D, VT, false>;
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::SMEM));
    int per_sm = 0;
    SANIC_CUDA_CHECK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, (size_t)Cfg<D>::SMEM));
    if (per_sm < 1) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "attn_decode_streamk: the kernel does not fit on an SM");
    int* counters = (int*)(p.partials + (size_t)p.batch * p.q_heads * p.n_splits * (D + 2));
    Exchange none{};
    cudaError_t le = launch_pdl(kern, dim3(ctx->sm_count * per_sm), dim3(128), (size_t)Cfg<D>::SMEM, st, p, counters, ctx->status_dev,
                                x ? *x : none, x ? 1 : 0);
    if (le != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("attn_decode_streamk: ") + cudaGetErrorString(le));
    return SANIC_OK;
}
int32_t streamk_validate_and_launch(sanic_ctx* ctx, const sanic_decode_params* p, cudaStream_t st, const Exchange* x) {
    int32_t rc = host_validate(ctx, p);
    if (rc != SANIC_OK) return rc;
    sanic_set_device(ctx);
    if (p->head_dim == 128) return p->v_transposed ? launch_streamk<128, true>(ctx, *p, st, x) : launch_streamk<128, false>(ctx, *p, st, x);
    return p->v_transposed ? launch_streamk<64, true>(ctx, *p, st, x) : launch_streamk<64, false>(ctx, *p, st, x);
}
}  // namespace

extern "C" {

// Partial slots per row the stream-K form needs: a group is crossed by at most ceil(resident CTAs / groups) + 1 ranges.
int32_t sanic_attn_decode_streamk_slots(sanic_ctx* ctx, int32_t batch, int32_t kv_heads, int32_t head_dim) {
    if (!ctx || batch <= 0 || kv_heads <= 0) return 1;
    const int per_sm = (head_dim == 128) ? 2 : 3;       // resident CTAs per SM by shared memory (an upper bound is all that matters)
    const long long G = (long long)ctx->sm_count * (per_sm + 1), groups = (long long)batch * kv_heads;
    return (int32_t)((G + groups - 1) / groups + 2);
}

int32_t sanic_attn_decode_streamk(sanic_ctx* ctx, const sanic_decode_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    return streamk_validate_and_launch(ctx, p, (cudaStream_t)stream, nullptr);
}

size_t sanic_peer_exchange_bytes_fused(int32_t rows, int32_t head_dim, int32_t nranks, int32_t groups) {
    if (rows <= 0 || head_dim <= 0 || nranks <= 0 || groups <= 0) return 0;
    return (xchg_flag_words(groups) + 2 * (size_t)nranks * rows * (head_dim + 2)) * 4;
}

int32_t sanic_splitkv_decode_step_fused(sanic_ctx* ctx, const sanic_decode_params* p, const sanic_peer_exchange* x, void* out,
                                        int32_t out_dtype, void* stream) {
    if (!ctx || !p || !x) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, out, "splitkv_decode_step_fused: out is required");
    SANIC_REQUIRE(ctx, x->nranks >= 1 && x->nranks <= 8 && x->rank >= 0 && x->rank < x->nranks, "splitkv_decode_step_fused: 1..8 ranks");
    SANIC_REQUIRE(ctx, x->epoch != 0, "splitkv_decode_step_fused: epochs start at 1 (the buffers start zeroed)");
    SANIC_REQUIRE(ctx, out_dtype == SANIC_BF16 || out_dtype == SANIC_F32, "splitkv_decode_step_fused: bad out dtype");
    Exchange e{};
    for (int q = 0; q < x->nranks; ++q) {
        SANIC_REQUIRE(ctx, x->buffers[q] && ((uintptr_t)x->buffers[q] % 16) == 0, "splitkv_decode_step_fused: missing or misaligned exchange buffer");
        e.buf[q] = (float*)x->buffers[q];
    }
    e.rank = x->rank; e.nranks = x->nranks; e.groups = p->batch * p->kv_heads;
    e.epoch = x->epoch; e.spin_limit = x->spin_limit ? x->spin_limit : (1u << 21);
    e.out = out; e.out_dtype = out_dtype;
    sanic_decode_params local = *p;
    local.out = nullptr;      // the local projection is meaningless before the cross-device merge
    if (!local.carrier_out) local.carrier_out = nullptr;
    // host_validate wants an output: the exchange is one
    sanic_decode_params chk = local;
    chk.out = out; chk.out_dtype = out_dtype;
    int32_t rc = host_validate(ctx, &chk);
    if (rc != SANIC_OK) return rc;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (p->head_dim == 128) return p->v_transposed ? launch_streamk<128, true>(ctx, local, st, &e) : launch_streamk<128, false>(ctx, local, st, &e);
    return p->v_transposed ? launch_streamk<64, true>(ctx, local, st, &e) : launch_streamk<64, false>(ctx, local, st, &e);
}

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
