// Decode-batch contraction y[b,o] = sum_k x[b,k] * W[o,k] for batch <= 16, HBM-bound.
//
// Weights are read exactly once, straight from global memory into MMA A-fragments with
// 128-bit (bf16) or 64-bit (int4) streaming loads; there is no shared-memory staging of
// the weight stream. The trick that makes direct loads coalesced: the k index of an
// m16n8k16 MMA may be permuted freely as long as A and B use the same permutation, so
// each thread takes 8 CONSECUTIVE k values of its row (one 16-byte load) and feeds them
// to two MMA steps; the activation fragment is loaded with the matching permutation.
//
// int4 (group-quantised, reference tests/metal.rs:1224-1236, nibble format
// src/emit_metal.rs:179-181): a nibble u = q + 8 becomes the bf16 value 128 + u by one
// lop3 (0x4300 | u is exactly 128 + u in bf16), i.e. q + 136. One k=64 group is four
// MMA steps into a fresh accumulator c; a second MMA chain against an all-ones A
// fragment gives c1 = sum_k x, and the group contributes scale * (c - 136 * c1). The
// scale is applied in f32 at the group boundary, as the derived carrier has it (the
// scale is pure axis structure).
//
// Work split: one CTA = 16 output rows (x 2 matrices for the silu(a)*b pair), its 8
// warps take contiguous K ranges and are summed in a fixed order through shared memory.
// When there are too few row tiles to fill the SMs, a thread-block cluster of 2-8 CTAs
// shares a tile, splits K, and rank 0 adds the peers' sums in rank order through
// distributed shared memory. Results are deterministic.
//
// Fusions that remove launches from a decode step:
//   * NORM: the producer cone of the activations (RMSNorm of the f32 residual stream) is
//     inlined: every CTA recomputes the row norms (a few KB from L2) and builds its bf16
//     activation fragments as bf16((x*g) * (1/den)) on the fly.
//   * ROPE_CACHE epilogue: for the q/k/v projections the CTA's 16 rows are the rotate-half
//     partners (d, d + D/2) of one head, so the epilogue rotates them and writes q, the K
//     cache row and the V cache column of the current position in place.
// Launched with programmatic dependent launch: weight prefetch runs before the wait.
#include "decode_step.cuh"
#include "gemv_body.cuh"

namespace {
using namespace sanic;
using namespace sanic::gemv;

// MINB: resident blocks per SM the register allocation is held to. A block is one 16-row tile, every warp's part of it a
// single batch of loads, so what hides the loads' latency is the number of resident blocks: three (80 registers) take the
// int4 lm_head from 81 to 68 us at batch 1; the short contractions lose with fewer registers (3.5 -> 4.2 us) and keep two.
template <bool W4, int NT, bool DUAL, bool NORM, int MINB = 2>
__global__ void __launch_bounds__(GW * 32, MINB) gemv_mma_kernel(const uint16_t* __restrict__ x, int batch, int K,
                                                           SegTable segs, int n_segments, int out_dtype, int epilogue,
                                                           const float* residual, Fused fz, int KS) {
    __shared__ float scratch[scratch_floats<NT, DUAL>()];
    gemv_tile<W4, NT, DUAL, NORM>(x, batch, K, segs, n_segments, out_dtype, epilogue, residual, fz, KS, (int)blockIdx.x, true, scratch);
}

template <bool W4, int NT, bool DUAL, bool NORM>
int32_t launch(sanic_ctx* ctx, const sanic_gemv_params& p, const SegTable& segs, const Fused& fz, int tiles, cudaStream_t st) {
    // Few row tiles cannot fill 148 SMs: split K over a cluster of KS CTAs per tile (each warp keeps
    // at least one 64-block of K).
    int KS = 1;
    const int nblk = p.K / 64;
    static const int ks_cap = getenv("SANIC_GEMV_KS") ? atoi(getenv("SANIC_GEMV_KS")) : 1;   // tuning knob: measured no gain on B200 at decode shapes, so off by default
    while (KS < ks_cap && tiles * KS < 2 * ctx->sm_count && nblk / (KS * 2) >= GW) KS *= 2;
    static const bool pdl = (getenv("SANIC_NO_PDL") == nullptr);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * KS); cfg.blockDim = dim3(GW * 32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) { attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization; attr[na].val.programmaticStreamSerializationAllowed = 1; ++na; }
    if (KS > 1) { attr[na].id = cudaLaunchAttributeClusterDimension; attr[na].val.clusterDim.x = KS; attr[na].val.clusterDim.y = 1; attr[na].val.clusterDim.z = 1; ++na; }
    cfg.attrs = attr; cfg.numAttrs = na;
    cudaError_t e;
    if (W4 && NT == 1 && !DUAL && !NORM && KS == 1 && p.K <= 2048 && tiles >= 8 * ctx->sm_count)
        e = cudaLaunchKernelEx(&cfg, gemv_mma_kernel<W4, NT, DUAL, NORM, (W4 && NT == 1 && !DUAL && !NORM) ? 3 : 2>, (const uint16_t*)p.x, p.batch,
                               p.K, segs, p.n_segments, p.out_dtype, p.epilogue, p.residual, fz, KS);
    else
        e = cudaLaunchKernelEx(&cfg, gemv_mma_kernel<W4, NT, DUAL, NORM>, (const uint16_t*)p.x, p.batch, p.K, segs,
                               p.n_segments, p.out_dtype, p.epilogue, p.residual, fz, KS);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemv: ") + cudaGetErrorString(e));
    return SANIC_OK;
}
template <bool W4, int NT, bool DUAL>
int32_t launch_n(sanic_ctx* ctx, const sanic_gemv_params& p, const SegTable& segs, const Fused& fz, int tiles, cudaStream_t st) {
    return fz.norm_x ? launch<W4, NT, DUAL, true>(ctx, p, segs, fz, tiles, st) : launch<W4, NT, DUAL, false>(ctx, p, segs, fz, tiles, st);
}
}  // namespace

extern "C" int32_t sanic_gemv(sanic_ctx* ctx, const sanic_gemv_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SegTable segs;
    Fused fz;
    int tiles = 0;
    int32_t rc = host_prepare(ctx, p, segs, fz, tiles);
    if (rc != SANIC_OK) return rc;
    const bool dual = p->epilogue == SANIC_EPI_SILU_MUL;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    const bool w4 = p->weight_dtype == SANIC_I4;
    const bool wide = p->batch > 8;
    // batch > 8: the contraction fed through a shared-memory ring by bulk copies keeps twice the bytes in flight
    // (SANIC_GEMV_RING=0 keeps the register-staged kernel, for A/B timing)
    static const bool ring = !(getenv("SANIC_GEMV_RING") && getenv("SANIC_GEMV_RING")[0] == '0');
    if (wide && ring && !p->norm_x) {
        rc = sanic::step::gemv_ring(ctx, p, st);
        if (rc != SANIC_ERR_UNSUPPORTED) return rc;
    }
    if (dual) {
        if (w4) return wide ? launch_n<true, 2, true>(ctx, *p, segs, fz, tiles, st) : launch_n<true, 1, true>(ctx, *p, segs, fz, tiles, st);
        return wide ? launch_n<false, 2, true>(ctx, *p, segs, fz, tiles, st) : launch_n<false, 1, true>(ctx, *p, segs, fz, tiles, st);
    }
    if (w4) return wide ? launch_n<true, 2, false>(ctx, *p, segs, fz, tiles, st) : launch_n<true, 1, false>(ctx, *p, segs, fz, tiles, st);
    return wide ? launch_n<false, 2, false>(ctx, *p, segs, fz, tiles, st) : launch_n<false, 1, false>(ctx, *p, segs, fz, tiles, st);
}
