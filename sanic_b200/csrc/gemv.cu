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
// warps take contiguous K ranges and are summed in a fixed order through shared memory,
// so results are deterministic.
#include "common.cuh"

namespace {
using namespace sanic;

constexpr int GW = 8;  // warps per CTA

struct SegTable {
    const void* w[3];
    const uint16_t* scales[3];
    void* out[3];
    int rows[3];
    int tile_begin[4];
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t nib_pair(uint32_t w) {  // (w & 0x000F000F) | 0x43004300
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(0x000F000Fu), "r"(0x43004300u));
    return r;
}

template <bool W4, int NT, bool DUAL>
__global__ void __launch_bounds__(GW * 32) gemv_mma_kernel(const uint16_t* __restrict__ x, int batch, int K,
                                                           SegTable segs, int n_segments, int out_dtype, int epilogue,
                                                           const float* residual) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    int seg = 0;
    if (!DUAL) {
        while (seg + 1 < n_segments && (int)blockIdx.x >= segs.tile_begin[seg + 1]) ++seg;
    }
    const int row0 = ((int)blockIdx.x - segs.tile_begin[seg]) * 16;
    constexpr int NM = DUAL ? 2 : 1;

    float acc[NM][NT][4];
#pragma unroll
    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[mI][j][0] = acc[mI][j][1] = acc[mI][j][2] = acc[mI][j][3] = 0.0f;

    const int nblk = K / 64;
    const int b0 = (warp * nblk) / GW, b1 = ((warp + 1) * nblk) / GW;
    const uint16_t* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = (8 * j + g) < batch;
        xrow[j] = x + (size_t)(xok[j] ? (8 * j + g) : 0) * K;
    }

    if (!W4) {
        const uint16_t* wr[NM][2];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            const uint16_t* W = (const uint16_t*)segs.w[DUAL ? mI : seg];
            wr[mI][0] = W + (size_t)(row0 + g) * K;
            wr[mI][1] = W + (size_t)(row0 + g + 8) * K;
        }
        constexpr int U = DUAL ? 2 : 4;
        int blk = b0;
        for (; blk + U <= b1; blk += U) {
            uint4 a[U][NM][2][2];
            uint4 xb[U][NT][2];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                int kb = (blk + u) * 64;
#pragma unroll
                for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        a[u][mI][r][0] = ldg_stream16(wr[mI][r] + kb + t * 8);
                        a[u][mI][r][1] = ldg_stream16(wr[mI][r] + kb + 32 + t * 8);
                    }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                int kb = (blk + u) * 64;
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    xb[u][j][0] = xok[j] ? __ldg((const uint4*)(xrow[j] + kb + t * 8)) : make_uint4(0, 0, 0, 0);
                    xb[u][j][1] = xok[j] ? __ldg((const uint4*)(xrow[j] + kb + 32 + t * 8)) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            const uint4& r0 = a[u][mI][0][hf];
                            const uint4& r1 = a[u][mI][1][hf];
                            const uint4& xv = xb[u][j][hf];
                            mma_bf16_16816(acc[mI][j], r0.x, r1.x, r0.y, r1.y, xv.x, xv.y);
                            mma_bf16_16816(acc[mI][j], r0.z, r1.z, r0.w, r1.w, xv.z, xv.w);
                        }
        }
        for (; blk < b1; ++blk) {
            int kb = blk * 64;
#pragma unroll
            for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    uint4 r0 = ldg_stream16(wr[mI][0] + kb + hf * 32 + t * 8);
                    uint4 r1 = ldg_stream16(wr[mI][1] + kb + hf * 32 + t * 8);
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        uint4 xv = xok[j] ? __ldg((const uint4*)(xrow[j] + kb + hf * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
                        mma_bf16_16816(acc[mI][j], r0.x, r1.x, r0.y, r1.y, xv.x, xv.y);
                        mma_bf16_16816(acc[mI][j], r0.z, r1.z, r0.w, r1.w, xv.z, xv.w);
                    }
                }
        }
    } else {
        const int G = K / 64;  // groups per row
        const uint8_t* wr[NM][2];
        const uint16_t* sr[NM][2];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            const uint8_t* W = (const uint8_t*)segs.w[DUAL ? mI : seg];
            const uint16_t* S = segs.scales[DUAL ? mI : seg];
            wr[mI][0] = W + (size_t)(row0 + g) * (K / 2);
            wr[mI][1] = W + (size_t)(row0 + g + 8) * (K / 2);
            sr[mI][0] = S + (size_t)(row0 + g) * G;
            sr[mI][1] = S + (size_t)(row0 + g + 8) * G;
        }
        constexpr int U = DUAL ? 2 : 4;
        const uint32_t ONES = 0x3F803F80u;
        auto do_group = [&](const uint2 (&wv)[NM][2], const float (&sc)[NM][2], int blk) {
            int kb = blk * 64 + t * 16;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint4 xa = xok[j] ? __ldg((const uint4*)(xrow[j] + kb)) : make_uint4(0, 0, 0, 0);
                uint4 xc = xok[j] ? __ldg((const uint4*)(xrow[j] + kb + 8)) : make_uint4(0, 0, 0, 0);
                // activation pairs matching the nibble pairing (n_i, n_{i+4})
                uint32_t bA0 = prmt(xa.x, xa.z, 0x5410), bA1 = prmt(xa.x, xa.z, 0x7632);
                uint32_t bA2 = prmt(xa.y, xa.w, 0x5410), bA3 = prmt(xa.y, xa.w, 0x7632);
                uint32_t bC0 = prmt(xc.x, xc.z, 0x5410), bC1 = prmt(xc.x, xc.z, 0x7632);
                uint32_t bC2 = prmt(xc.y, xc.w, 0x5410), bC3 = prmt(xc.y, xc.w, 0x7632);
                float c1[4] = {0, 0, 0, 0};
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bA0, bA1);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bA2, bA3);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bC0, bC1);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bC2, bC3);
#pragma unroll
                for (int mI = 0; mI < NM; ++mI) {
                    uint32_t w0a = wv[mI][0].x, w0b = wv[mI][0].y, w1a = wv[mI][1].x, w1b = wv[mI][1].y;
                    float c[4] = {0, 0, 0, 0};
                    mma_bf16_16816(c, nib_pair(w0a), nib_pair(w1a), nib_pair(w0a >> 4), nib_pair(w1a >> 4), bA0, bA1);
                    mma_bf16_16816(c, nib_pair(w0a >> 8), nib_pair(w1a >> 8), nib_pair(w0a >> 12), nib_pair(w1a >> 12), bA2, bA3);
                    mma_bf16_16816(c, nib_pair(w0b), nib_pair(w1b), nib_pair(w0b >> 4), nib_pair(w1b >> 4), bC0, bC1);
                    mma_bf16_16816(c, nib_pair(w0b >> 8), nib_pair(w1b >> 8), nib_pair(w0b >> 12), nib_pair(w1b >> 12), bC2, bC3);
                    acc[mI][j][0] = fmaf(sc[mI][0], fmaf(-136.0f, c1[0], c[0]), acc[mI][j][0]);
                    acc[mI][j][1] = fmaf(sc[mI][0], fmaf(-136.0f, c1[1], c[1]), acc[mI][j][1]);
                    acc[mI][j][2] = fmaf(sc[mI][1], fmaf(-136.0f, c1[2], c[2]), acc[mI][j][2]);
                    acc[mI][j][3] = fmaf(sc[mI][1], fmaf(-136.0f, c1[3], c[3]), acc[mI][j][3]);
                }
            }
        };
        int blk = b0;
        for (; blk + U <= b1; blk += U) {
            uint2 wv[U][NM][2];
            float sc[U][NM][2];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        wv[u][mI][r] = ldg_stream8(wr[mI][r] + (size_t)(blk + u) * 32 + t * 8);
                        sc[u][mI][r] = bf16_to_f32(__ldg(sr[mI][r] + blk + u));
                    }
#pragma unroll
            for (int u = 0; u < U; ++u) do_group(wv[u], sc[u], blk + u);
        }
        for (; blk < b1; ++blk) {
            uint2 wv[NM][2];
            float sc[NM][2];
#pragma unroll
            for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    wv[mI][r] = ldg_stream8(wr[mI][r] + (size_t)blk * 32 + t * 8);
                    sc[mI][r] = bf16_to_f32(__ldg(sr[mI][r] + blk));
                }
            do_group(wv, sc, blk);
        }
    }

    // deterministic cross-warp sum: red[warp][matrix][row 0..15][col 0..8*NT)
    __shared__ float red[GW][NM][16][8 * NT + 1];
#pragma unroll
    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            red[warp][mI][g][8 * j + 2 * t] = acc[mI][j][0];
            red[warp][mI][g][8 * j + 2 * t + 1] = acc[mI][j][1];
            red[warp][mI][g + 8][8 * j + 2 * t] = acc[mI][j][2];
            red[warp][mI][g + 8][8 * j + 2 * t + 1] = acc[mI][j][3];
        }
    __syncthreads();
    for (int idx = tid; idx < 16 * batch; idx += GW * 32) {
        int n = idx / 16, r = idx % 16;  // consecutive threads -> consecutive rows (contiguous in out[n][row])
        float v[NM];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            float s = 0.0f;
#pragma unroll
            for (int w = 0; w < GW; ++w) s += red[w][mI][r][n];
            v[mI] = s;
        }
        float y = v[0];
        if (DUAL) {  // silu(a) * b = (a * 1/(1+exp(-a))) * b  (reference src/ir.rs:1500-1509)
            float sig = 1.0f / (1.0f + expf(-v[0]));
            y = (v[0] * sig) * v[NM - 1];
        }
        int rows = segs.rows[seg];
        size_t oi = (size_t)n * rows + row0 + r;
        if (epilogue == SANIC_EPI_RESIDUAL_ADD) y = residual[oi] + y;
        if (out_dtype == SANIC_BF16) ((uint16_t*)segs.out[seg])[oi] = f32_to_bf16_bits(y);
        else ((float*)segs.out[seg])[oi] = y;
    }
}

template <bool W4, int NT, bool DUAL>
int32_t launch(sanic_ctx* ctx, const sanic_gemv_params& p, const SegTable& segs, int tiles, cudaStream_t st) {
    gemv_mma_kernel<W4, NT, DUAL><<<tiles, GW * 32, 0, st>>>((const uint16_t*)p.x, p.batch, p.K, segs, p.n_segments,
                                                             p.out_dtype, p.epilogue, p.residual);
    SANIC_LAUNCH_CHECK(ctx, "gemv");
    return SANIC_OK;
}
}  // namespace

extern "C" int32_t sanic_gemv(sanic_ctx* ctx, const sanic_gemv_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->x && p->batch >= 1 && p->batch <= 16, "gemv: batch must be in [1, 16]");
    SANIC_REQUIRE(ctx, p->K >= 64 && p->K % 64 == 0, "gemv: K must be a multiple of 64");
    SANIC_REQUIRE(ctx, p->n_segments >= 1 && p->n_segments <= 3, "gemv: 1..3 weight segments");
    if (p->weight_dtype != SANIC_BF16 && p->weight_dtype != SANIC_I4)
        return sanic_fail(ctx, SANIC_ERR_DTYPE, "gemv: weights must be bf16 or int4");
    SANIC_REQUIRE(ctx, p->weight_dtype != SANIC_I4 || p->group == 64, "gemv: int4 group size must be 64");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_F32 || p->out_dtype == SANIC_BF16, "gemv: output must be f32 or bf16");
    SANIC_REQUIRE(ctx, ((uintptr_t)p->x % 16) == 0, "gemv: activations must be 16-byte aligned");
    bool dual = p->epilogue == SANIC_EPI_SILU_MUL;
    SANIC_REQUIRE(ctx, !dual || (p->n_segments == 2 && p->rows[0] == p->rows[1]), "gemv: silu-mul needs two equal segments");
    SANIC_REQUIRE(ctx, p->epilogue != SANIC_EPI_RESIDUAL_ADD || (p->residual && p->n_segments == 1),
                  "gemv: residual-add needs one segment and a residual");
    SegTable segs{};
    int tiles = 0;
    for (int i = 0; i < p->n_segments; ++i) {
        SANIC_REQUIRE(ctx, p->w[i] && p->rows[i] > 0 && p->rows[i] % 16 == 0,
                      "gemv: segment rows must be a positive multiple of 16");
        SANIC_REQUIRE(ctx, p->out[i] || (dual && i == 1), "gemv: null output");
        SANIC_REQUIRE(ctx, ((uintptr_t)p->w[i] % 16) == 0, "gemv: weights must be 16-byte aligned");
        SANIC_REQUIRE(ctx, p->weight_dtype != SANIC_I4 || p->scales[i], "gemv: int4 weights need scales");
        segs.w[i] = p->w[i];
        segs.scales[i] = (const uint16_t*)p->scales[i];
        segs.out[i] = p->out[i];
        segs.rows[i] = p->rows[i];
        segs.tile_begin[i] = tiles;
        if (!dual || i == 0) tiles += p->rows[i] / 16;
    }
    for (int i = p->n_segments; i < 4; ++i) segs.tile_begin[i] = tiles;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    bool w4 = p->weight_dtype == SANIC_I4;
    bool wide = p->batch > 8;
    if (dual) {
        if (w4) return wide ? launch<true, 2, true>(ctx, *p, segs, tiles, st) : launch<true, 1, true>(ctx, *p, segs, tiles, st);
        return wide ? launch<false, 2, true>(ctx, *p, segs, tiles, st) : launch<false, 1, true>(ctx, *p, segs, tiles, st);
    }
    if (w4) return wide ? launch<true, 2, false>(ctx, *p, segs, tiles, st) : launch<true, 1, false>(ctx, *p, segs, tiles, st);
    return wide ? launch<false, 2, false>(ctx, *p, segs, tiles, st) : launch<false, 1, false>(ctx, *p, segs, tiles, st);
}
