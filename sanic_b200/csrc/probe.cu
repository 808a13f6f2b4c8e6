// Measured device facts the schedules are planned with: what DeviceSpecs carries next to the datasheet figures
// (reference src/cost.rs:33-119: `DeviceSpecs`, fitted per device; src/compile.rs:1348-1630 times candidates in
// context). Two probes, both tiny and bounded:
//
//   sfu     exponentials per clock per SM. The online-softmax fold at head_dim 64 issues 16,384 `ex2` per 128x128 score
//           tile next to 512 clocks of tensor-core work, so this rate, and how much of the warps' other instructions
//           (scale, row sum, bf16 pack) the SM overlaps with it, is the bound of the prefill kernel. Mode 0 issues only
//           the exponentials from registers; modes 1-3 add, per element, the FMA that scales and shifts the score, the
//           add of the row sum and the bf16x2 pack of the result: exactly the softmax warp's inner loop. Modes 4 and 5 are
//           mode 3 with every fourth / every second pair of exponentials computed on the FMA pipe (a cubic after range
//           reduction) instead of the SFU: what moving part of the load off the SFU buys. Modes 6-8 take the exponentials
//           of a pair as ONE packed half-precision instruction (arguments rounded to f16): 6 = scale, convert and the
//           packed exponential alone, 7 = + unpack to f32 for the row sum and the bf16x2 pack, 8 = + unpack and row sum,
//           the pair kept as f16. Modes 9 and 10 are mode 3 with the row maximum taken in the same loop: one three-input
//           max per pair, or two two-input ones.
//   stream  a plain read-only sweep of a buffer (16-byte loads, every SM): the HBM read rate a fold can be held to.
#include "common.cuh"

namespace {
using namespace sanic;

__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float max3(float a, float b, float c) { float y; asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c)); return y; }

// exp2 of a pair on the FMA pipe: round to the nearest integer with the 1.5 * 2^23 trick, a cubic on the remainder in
// [-0.5, 0.5] (relative error 1e-4: inside the bf16 rounding the result gets anyway), and the integer part added into
// the exponent field. Packed f32x2 arithmetic: 3 adds and 3 FMAs per pair, plus one integer multiply-add per element.
__device__ __forceinline__ void ex2_poly2(float& p0, float& p1, float x0, float x1) {
    const float MAGIC = 12582912.0f;     // 1.5 * 2^23
    float t0, t1, r0, r1, f0, f1, q0, q1;
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tadd.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(t0), "=f"(t1) : "f"(x0), "f"(x1), "f"(MAGIC));
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tadd.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(r0), "=f"(r1) : "f"(t0), "f"(t1), "f"(-MAGIC));
    asm("{\n\t.reg .b64 a, b, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tsub.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(f0), "=f"(f1) : "f"(x0), "f"(x1), "f"(r0), "f"(r1));
    const float C3 = 0.0555041087f, C2 = 0.2402265069f, C1 = 0.6931471806f;
    asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %4};\n\tmov.b64 c, {%5, %5};\n\tfma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(q0), "=f"(q1) : "f"(f0), "f"(f1), "f"(C3), "f"(C2));
    asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%6, %6};\n\tfma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(q0), "=f"(q1) : "f"(q0), "f"(q1), "f"(f0), "f"(f1), "f"(C1));
    asm("{\n\t.reg .b64 a, b, c, d;\n\tmov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%6, %6};\n\tfma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(q0), "=f"(q1) : "f"(q0), "f"(q1), "f"(f0), "f"(f1), "f"(1.0f));
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// exp2 of a pair as one packed half-precision SFU instruction: the arguments are rounded to f16 first
__device__ __forceinline__ uint32_t ex2_h2(float x0, float x1) {
    uint32_t h, y;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(x1), "f"(x0));
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(h));
    return y;
}
__device__ __forceinline__ void unpack_h2(uint32_t h, float& lo, float& hi) {
    asm("{\n\t.reg .b16 l, u;\n\tmov.b32 {l, u}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, u;\n\t}" : "=f"(lo), "=f"(hi) : "r"(h));
}

template <int MODE>
__global__ void probe_sfu_kernel(float* out, const float* in, long long* clk, int iters) {
    float r[128];
    for (int i = 0; i < 128; ++i) r[i] = in[(threadIdx.x * 128 + i) % 4096];
    const float sl2 = in[0], msub = in[1];
    float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint32_t acc = 0;
    float mx3[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            float a = r[2 * i], b = r[2 * i + 1];
            if (MODE >= 1) { a = fmaf(a, sl2, -msub); b = fmaf(b, sl2, -msub); }
            constexpr int M = MODE >= 9 ? 3 : MODE;      // modes 9 and 10 are mode 3 plus the maximum
            if (MODE == 9) mx3[i & 3] = max3(mx3[i & 3], a, b);                              // a row maximum next to the loop
            if (MODE == 10) { mx3[i & 3] = fmaxf(mx3[i & 3], a); mx3[(i + 2) & 3] = fmaxf(mx3[(i + 2) & 3], b); }
            if (MODE >= 6 && MODE <= 8) {
                // modes 6-8: one packed f16x2 exponential per pair; 7 unpacks it for the f32 row sum and packs bf16,
                // 8 unpacks for the row sum and keeps the f16 pair
                const uint32_t h = ex2_h2(a, b);
                if (MODE >= 7) {
                    float p0, p1;
                    unpack_h2(h, p0, p1);
                    sums[(2 * i) & 7] += p0; sums[(2 * i + 1) & 7] += p1;
                    pk[i] = (MODE == 7) ? pack_bf16x2(p0, p1) : h;
                } else pk[i] = h;
                continue;
            }
            float p0, p1;
            // modes 4 and 5: every fourth / every second pair takes its exponentials on the FMA pipe instead of the SFU
            if ((M == 4 && (i & 3) == 3) || (M == 5 && (i & 1) == 1)) ex2_poly2(p0, p1, a, b);
            else { p0 = ex2(a); p1 = ex2(b); }
            if (M >= 2) { sums[(2 * i) & 7] += p0; sums[(2 * i + 1) & 7] += p1; }
            pk[i] = (M >= 3) ? pack_bf16x2(p0, p1) : (__float_as_uint(p0) ^ __float_as_uint(p1));
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) acc ^= pk[i];
#pragma unroll
        for (int i = 0; i < 128; ++i) r[i] += __uint_as_float(acc & 1);   // a dependence that keeps the loop from collapsing
    }
    const long long t1 = clock64();
    float s = 0;
    for (int i = 0; i < 8; ++i) s += sums[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s + __uint_as_float(acc) + r[5] + fmaxf(fmaxf(mx3[0], mx3[1]), fmaxf(mx3[2], mx3[3]));
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
    SANIC_REQUIRE(ctx, warps_per_sm >= 1 && warps_per_sm <= 32 && mode >= 0 && mode <= 10 && iters >= 1 && iters <= 10000,
                  "probe_sfu: warps per SM in [1, 32], mode in [0, 10], iterations in [1, 10000]");
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
        else if (mode == 3) probe_sfu_kernel<3><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 4) probe_sfu_kernel<4><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 5) probe_sfu_kernel<5><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 6) probe_sfu_kernel<6><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 7) probe_sfu_kernel<7><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 8) probe_sfu_kernel<8><<<g, b, 0, st>>>(out, in, clk, iters);
        else if (mode == 9) probe_sfu_kernel<9><<<g, b, 0, st>>>(out, in, clk, iters);
        else probe_sfu_kernel<10><<<g, b, 0, st>>>(out, in, clk, iters);
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
