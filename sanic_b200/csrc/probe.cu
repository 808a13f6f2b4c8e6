// Measured device facts the schedules are planned with: what DeviceSpecs carries next to the datasheet figures
// (reference src/cost.rs:33-119: `DeviceSpecs`, fitted per device; src/compile.rs:1348-1630 times candidates in
// context). Two probes, both tiny and bounded:
//
//   sfu     exponentials per clock per SM. The online-softmax fold at head_dim 64 issues 16,384 `ex2` per 128x128 score
//           tile next to 512 clocks of tensor-core work, so this rate, and how much of the warps' other instructions
//           (scale, row sum, bf16 pack) the SM overlaps with it, is the bound of the prefill kernel. Mode 0 issues only
//           the exponentials from registers; modes 1-3 add, per element, the FMA that scales and shifts the score, the
//           add of the row sum and the bf16x2 pack of the result: exactly the softmax warp's inner loop.
//   stream  a plain read-only sweep of a buffer (16-byte loads, every SM): the HBM read rate a fold can be held to.
#include "common.cuh"

namespace {
using namespace sanic;

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

template <int MODE>
__global__ void probe_sfu_kernel(float* out, const float* in, long long* clk, int iters) {
    float r[128];
    for (int i = 0; i < 128; ++i) r[i] = in[(threadIdx.x * 128 + i) % 4096];
    const float sl2 = in[0], msub = in[1];
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t acc = 0;
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            float a = r[2 * i], b = r[2 * i + 1];
            if (MODE >= 1) { a = fmaf(a, sl2, -msub); b = fmaf(b, sl2, -msub); }
            const float p0 = ex2(a), p1 = ex2(b);
            if (MODE >= 2) { sums[(2 * i) & 7] += p0; sums[(2 * i + 1) & 7] += p1; }
            pk[i] = (MODE >= 3) ? pack_bf16x2(p0, p1) : (__float_as_uint(p0) ^ __float_as_uint(p1));
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) acc ^= pk[i];
#pragma unroll
        for (int i = 0; i < 128; ++i) r[i] += __uint_as_float(acc & 1);   // a dependence that keeps the loop from collapsing
    }
    const long long t1 = clock64();
    float s = 0;
    for (int i = 0; i < 8; ++i) s += sums[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s + __uint_as_float(acc) + r[5];
    if (threadIdx.x == 0 && blockIdx.x == 0) clk[0] = (t1 - t0) / iters;
}

__global__ void probe_stream_kernel(const uint4* __restrict__ src, size_t n16, unsigned* sink) {
    unsigned acc = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = ldg_stream16(src + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9E3779B9u) *sink = acc;      // never true for the probe's data; keeps the loads alive
}
}  // namespace

extern "C" {

int32_t sanic_probe_sfu(sanic_ctx* ctx, int32_t warps_per_sm, int32_t mode, int32_t iters, void* stream, double* exp_per_clk_per_sm,
                        double* clk_per_128_per_warp) {
    if (!ctx || !exp_per_clk_per_sm) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, warps_per_sm >= 1 && warps_per_sm <= 32 && mode >= 0 && mode <= 3 && iters >= 1 && iters <= 10000,
                  "probe_sfu: warps per SM in [1, 32], mode in [0, 3], iterations in [1, 10000]");
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    float *out = nullptr, *in = nullptr;
    long long* clk = nullptr;
    cudaError_t e = cudaMalloc(&out, (size_t)ctx->sm_count * 1024 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&in, 4096 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&clk, sizeof(long long));
    if (e == cudaSuccess) e = cudaMemsetAsync(in, 0, 4096 * sizeof(float), st);
    long long h = 0;
    for (int rep = 0; rep < 2 && e == cudaSuccess; ++rep) {       // the first launch warms the instruction cache
        const dim3 g(ctx->sm_count), b(warps_per_sm * 32);
        if (mode == 0) probe_sfu_kernel<0><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 1) probe_sfu_kernel<1><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 2) probe_sfu_kernel<2><<<g, b, 0, st>>>(out, in, clk, iters);
        else probe_sfu_kernel<3><<<g, b, 0, st>>>(out, in, clk, iters);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    }
    if (e == cudaSuccess) e = cudaMemcpy(&h, clk, sizeof(long long), cudaMemcpyDeviceToHost);
    cudaFree(out); cudaFree(in); cudaFree(clk);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("probe_sfu: ") + cudaGetErrorString(e));
    if (h <= 0) return sanic_fail(ctx, SANIC_ERR_CUDA, "probe_sfu: the clock did not advance");
    // one iteration of one warp is 128 elements on each of its 32 lanes
    *exp_per_clk_per_sm = (double)warps_per_sm * 128.0 * 32.0 / (double)h;
    if (clk_per_128_per_warp) *clk_per_128_per_warp = (double)h;
    return SANIC_OK;
}

int32_t sanic_probe_stream(sanic_ctx* ctx, const void* buffer, size_t bytes, int32_t repeats, void* stream, double* gb_per_s) {
    if (!ctx || !buffer || !gb_per_s) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, bytes >= (1u << 20) && bytes % 16 == 0 && ((uintptr_t)buffer % 16) == 0 && repeats >= 1 && repeats <= 1000,
                  "probe_stream: at least 1 MiB, 16-byte aligned and sized, 1..1000 repeats");
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t e = cudaMalloc(&sink, sizeof(unsigned));
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    float best = 1e30f;
    for (int r = 0; r < repeats + 1 && e == cudaSuccess; ++r) {
        cudaEventRecord(e0, st);
        probe_stream_kernel<<<ctx->sm_count * 8, 512, 0, st>>>((const uint4*)buffer, bytes / 16, sink);
        cudaEventRecord(e1, st);
        e = cudaEventSynchronize(e1);
        float ms = 0.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        if (r > 0 && ms < best) best = ms;
    }
    if (sink) cudaFree(sink);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("probe_stream: ") + cudaGetErrorString(e));
    *gb_per_s = (double)bytes / ((double)best * 1e-3) / 1e9;
    return SANIC_OK;
}

}  // extern "C"
