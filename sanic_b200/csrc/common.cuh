// Shared host/device helpers for the sm_100a kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <string>

#include "../../include/sanic_b200.h"

struct sanic_ctx {
    int device = 0;
    int sm_count = 0;
    int max_smem = 0;
    int l2_bytes = 0;
    int cc_major = 0, cc_minor = 0;
    size_t hbm_bytes = 0;
    std::string err;
    // NCCL (resolved at run time; see nccl_merge.cu)
    void* nccl_lib = nullptr;
    void* nccl_comm = nullptr;
    int nccl_rank = 0, nccl_nranks = 1;
    // cached driver entry point for tensor-map encoding (gemm_rmsnorm.cu)
    void* encode_tiled = nullptr;
    // device-side status word in mapped pinned memory: kernels with bounded waits write a
    // nonzero code here, the host reads it without a synchronising copy
    int* status_host = nullptr;
    int* status_dev = nullptr;
    // device buffer of the GEMM's clock counters, non-null only inside sanic_gemm_rmsnorm_pair_profile
    unsigned long long* gemm_prof = nullptr;
};

namespace sanic {
// device-free structure checks of one stage (program.cu); `why` receives the refusal
int32_t stage_check(const sanic_stage_desc& s, std::string* why, bool pointers);
}
static inline int32_t sanic_fail(sanic_ctx* ctx, int32_t code, const std::string& msg) {
    if (ctx) ctx->err = msg;
    return code;
}
#define SANIC_CUDA_CHECK(ctx, call)                                                              \
    do {                                                                                         \
        cudaError_t _e = (call);                                                                 \
        if (_e != cudaSuccess)                                                                   \
            return sanic_fail((ctx), SANIC_ERR_CUDA,                                             \
                              std::string(#call) + ": " + cudaGetErrorString(_e));               \
    } while (0)
#define SANIC_LAUNCH_CHECK(ctx, what)                                                            \
    do {                                                                                         \
        cudaError_t _e = cudaGetLastError();                                                     \
        if (_e != cudaSuccess)                                                                   \
            return sanic_fail((ctx), SANIC_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(_e)); \
    } while (0)
#define SANIC_REQUIRE(ctx, cond, msg)                                                            \
    do {                                                                                         \
        if (!(cond)) return sanic_fail((ctx), SANIC_ERR_INVALID, std::string(msg));              \
    } while (0)

static inline int sanic_set_device(sanic_ctx* ctx) { return (int)cudaSetDevice(ctx->device); }

#ifdef __CUDACC__
namespace sanic {

// Programmatic dependent launch: a kernel launched this way may start while its predecessor in the
// stream drains. It must execute griddep_wait() before it touches memory the predecessor wrote
// (every kernel of a chain does, so completion stays transitive) and may call griddep_launch()
// early to let its own successor begin its prologue.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args... args) {
    static const bool pdl = (getenv("SANIC_NO_PDL") == nullptr);   // SANIC_NO_PDL=1: plain stream order (for A/B timing)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// ── typed loads / stores: bit-exact twins of scalar::round_to (reference src/scalar.rs:120-135) ──
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
    uint32_t b = __float_as_uint(f);
    if (f != f) return (uint16_t)((b >> 16) | 0x0040u);  // keep NaN quiet, keep its sign
    return (uint16_t)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
// Two f32 -> packed bf16x2 (lo in the low half). Hardware RNE; identical to the
// function above for every non-NaN input.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
// u32 saturating store of a non-negative real (reference src/emit_metal.rs:186-190).
__device__ __forceinline__ uint32_t f32_to_u32_sat(float f) {
    if (!(f > 0.0f)) return 0u;
    if (f >= 4294967296.0f) return 0xFFFFFFFFu;
    return (uint32_t)f;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte async copy global -> shared; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Streaming 16-byte / 8-byte global loads that bypass L1 allocation (weights and KV are read once).
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// The derived combine of an ExpShifted slot pair sharing max slot m (reference
// src/derive.rs:1700-1713): a side whose max is -inf is forced to weight 0.
struct MloScale { float ra, rb, m; };
__device__ __forceinline__ MloScale mlo_rescale(float ma, float mb) {
    MloScale s;
    s.m = fmaxf(ma, mb);
    s.ra = (ma > -INFINITY) ? expf(ma - s.m) : 0.0f;
    s.rb = (mb > -INFINITY) ? expf(mb - s.m) : 0.0f;
    return s;
}

}  // namespace sanic
#endif  // __CUDACC__
