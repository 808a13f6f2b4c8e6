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
// A thread-block cluster of 2-8 CTAs can share a tile, split K, and have rank 0 add the
// peers' sums in rank order through distributed shared memory; two CTAs per tile are the
// default for a K axis of 4096 or more with at most one tile per SM (the down projection).
// Results are deterministic. Three other forms take the shapes this split serves badly:
//   * batch 9-16: gemv_ring_kernel (decode_step.cu), weights through a shared-memory ring;
//   * one int4 matrix of at least 16 row tiles per SM with a plain store (the lm_head):
//     gemv_w4_rows_kernel below, a warp per 16-row tile;
//   * int4 silu(a)*b at K <= 2048 up to batch 8: gemv_w4_dual_team_kernel below, four warps
//     per dual tile.
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

// int4-g64 weights, batch <= 8, one matrix with many row tiles and a plain store (the lm_head): a WARP owns whole 16-row
// tiles. With a block per tile and the K axis split over its warps, a warp's share of a tile is one batch of loads and
// every tile pays a block barrier and a cross-warp sum; here a warp walks the K axis of its tile four groups at a time with
// the next four groups' loads (a 8-byte weight load per row and group: the four lanes of a row read one 32-byte sector; one
// 8-byte load of four scales per row) in flight under the arithmetic, accumulates alone and stores its 16 rows itself.
// What depends on the activations only is taken once per block: they are staged in shared memory as bf16 (norm applied),
// already in the order of the MMA's B fragments (the byte permutes that pair activations like the nibbles are paired), and
// the zero point's term, 136 x the sum of a group's activations, is kept per group (the four MMAs against ones that the
// tile-per-block form issues for every tile and group).
constexpr int WR_U = 4;
template <bool NORM, int NT>
__global__ void __launch_bounds__(GW * 32, 2) gemv_w4_rows_kernel(const uint16_t* __restrict__ x, int batch, int K, SegTable segs, int out_dtype,
                                                                 Fused fz, int tiles) {
    extern __shared__ __align__(16) unsigned char wr_smem[];
    float* scratch = (float*)wr_smem;                                 // row norms or deferred scales: 16 + 16 * GW floats
    const int G = K / 64, xpitch = K * 2 + 16;                        // rows 4 banks apart: conflict-free 16-byte reads by a quarter warp
    float2* gsum = (float2*)(wr_smem + 1024);                         // [K / 64][NT][4]: sums of columns 2t, 2t+1 (+ 8 per half) per group
    unsigned char* xs = wr_smem + 1024 + G * NT * 32;                 // [8 * NT][xpitch]: per group and lane quarter t, the 8 B-fragment registers
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    griddep_launch();
    griddep_wait();
    if (NORM) row_norms<false>(fz, batch, K, scratch);
    else if (fz.ds_partial) defer_scales<false>(fz, batch, scratch);        // the outputs' scale per batch row (deferred normaliser)
    for (int i = tid; i < batch * (K / 16); i += GW * 32) {
        const int n = i / (K / 16), c = i % (K / 16);     // c = 4 * group + t: 16 activations
        const uint16_t* xr = NORM ? nullptr : x + (size_t)n * K;
        const float* xf = NORM ? fz.norm_x + (size_t)n * K : nullptr;
        const uint4 xa = load_x8<NORM, false>(xr, xf, fz.norm_gamma, NORM ? scratch[n] : 1.0f, c * 16, true);
        const uint4 xc = load_x8<NORM, false>(xr, xf, fz.norm_gamma, NORM ? scratch[n] : 1.0f, c * 16 + 8, true);
        // activation pairs matching the nibble pairing (n_i, n_{i+4})
        uint4* dst = (uint4*)(xs + (size_t)n * xpitch + c * 32);
        dst[0] = make_uint4(prmt(xa.x, xa.z, 0x5410), prmt(xa.x, xa.z, 0x7632), prmt(xa.y, xa.w, 0x5410), prmt(xa.y, xa.w, 0x7632));
        dst[1] = make_uint4(prmt(xc.x, xc.z, 0x5410), prmt(xc.x, xc.z, 0x7632), prmt(xc.y, xc.w, 0x5410), prmt(xc.y, xc.w, 0x7632));
    }
    __syncthreads();
    bool xok[NT];
    const unsigned char* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = 8 * j + g < batch;
        xrow[j] = xs + (size_t)(xok[j] ? 8 * j + g : 0) * xpitch + t * 32;
    }
    // the B fragments of group u for batch columns 8j .. 8j+7
    auto x_frags = [&](int u, int j, uint32_t (&b)[8]) {
        const uint4 lo = xok[j] ? *(const uint4*)(xrow[j] + (size_t)u * 128) : make_uint4(0, 0, 0, 0);
        const uint4 hi = xok[j] ? *(const uint4*)(xrow[j] + (size_t)u * 128 + 16) : make_uint4(0, 0, 0, 0);
        b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w; b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
    };
    {
        const uint32_t ONES = 0x3F803F80u;
        for (int u = warp; u < G; u += GW) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint32_t b[8];
                x_frags(u, j, b);
                float c1[4] = {0, 0, 0, 0};
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[0], b[1]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[2], b[3]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[4], b[5]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[6], b[7]);
                if (g == 0) gsum[(u * NT + j) * 4 + t] = make_float2(c1[0], c1[1]);       // every row of c1 is the same
            }
        }
    }
    __syncthreads();
    const uint8_t* W = (const uint8_t*)segs.w[0];
    const uint16_t* S = segs.scales[0];
    const int rows = segs.rows[0];
    const bool scaled = !NORM && fz.ds_partial != nullptr;
    for (int tile = blockIdx.x * GW + warp; tile < tiles; tile += gridDim.x * GW) {
        const uint8_t* w0 = W + (size_t)(tile * 16 + g) * (K / 2) + t * 8;
        const uint8_t* w1 = w0 + (size_t)8 * (K / 2);
        const uint16_t* s0 = S + (size_t)(tile * 16 + g) * G;
        const uint16_t* s1 = s0 + (size_t)8 * G;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        uint2 wa[WR_U][2], sa[2];
#pragma unroll
        for (int u = 0; u < WR_U; ++u) { wa[u][0] = ldg_stream8(w0 + u * 32); wa[u][1] = ldg_stream8(w1 + u * 32); }
        sa[0] = ldg_stream8(s0); sa[1] = ldg_stream8(s1);
        for (int blk = 0; blk < G; blk += WR_U) {
            uint2 wn[WR_U][2], sn[2];
            const bool more = blk + WR_U < G;
            if (more) {
#pragma unroll
                for (int u = 0; u < WR_U; ++u) {
                    wn[u][0] = ldg_stream8(w0 + (size_t)(blk + WR_U + u) * 32);
                    wn[u][1] = ldg_stream8(w1 + (size_t)(blk + WR_U + u) * 32);
                }
                sn[0] = ldg_stream8(s0 + blk + WR_U); sn[1] = ldg_stream8(s1 + blk + WR_U);
            }
#pragma unroll
            for (int u = 0; u < WR_U; ++u) {
                const uint32_t sw0 = (u < 2) ? sa[0].x : sa[0].y, sw1 = (u < 2) ? sa[1].x : sa[1].y;
                const float sc0 = (u & 1) ? bf16hi(sw0) : bf16lo(sw0), sc1 = (u & 1) ? bf16hi(sw1) : bf16lo(sw1);
                const uint32_t a0 = wa[u][0].x, a1 = wa[u][0].y, c0 = wa[u][1].x, c1w = wa[u][1].y;
                const uint32_t f0 = nib_pair(a0), f1 = nib_pair(c0), f2 = nib_pair(a0 >> 4), f3 = nib_pair(c0 >> 4);
                const uint32_t f4 = nib_pair(a0 >> 8), f5 = nib_pair(c0 >> 8), f6 = nib_pair(a0 >> 12), f7 = nib_pair(c0 >> 12);
                const uint32_t h0 = nib_pair(a1), h1 = nib_pair(c1w), h2 = nib_pair(a1 >> 4), h3 = nib_pair(c1w >> 4);
                const uint32_t h4 = nib_pair(a1 >> 8), h5 = nib_pair(c1w >> 8), h6 = nib_pair(a1 >> 12), h7 = nib_pair(c1w >> 12);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    uint32_t b[8];
                    x_frags(blk + u, j, b);
                    const float2 cs = gsum[((blk + u) * NT + j) * 4 + t];
                    float c[4] = {0, 0, 0, 0};
                    mma_bf16_16816(c, f0, f1, f2, f3, b[0], b[1]);
                    mma_bf16_16816(c, f4, f5, f6, f7, b[2], b[3]);
                    mma_bf16_16816(c, h0, h1, h2, h3, b[4], b[5]);
                    mma_bf16_16816(c, h4, h5, h6, h7, b[6], b[7]);
                    acc[j][0] = fmaf(sc0, fmaf(-136.0f, cs.x, c[0]), acc[j][0]);
                    acc[j][1] = fmaf(sc0, fmaf(-136.0f, cs.y, c[1]), acc[j][1]);
                    acc[j][2] = fmaf(sc1, fmaf(-136.0f, cs.x, c[2]), acc[j][2]);
                    acc[j][3] = fmaf(sc1, fmaf(-136.0f, cs.y, c[3]), acc[j][3]);
                }
            }
            if (more) {
#pragma unroll
                for (int u = 0; u < WR_U; ++u) { wa[u][0] = wn[u][0]; wa[u][1] = wn[u][1]; }
                sa[0] = sn[0]; sa[1] = sn[1];
            }
        }
        // C fragment: rows g and g+8 of the tile, batch columns 8j + 2t and 8j + 2t + 1
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int n = 8 * j + 2 * t + (i & 1), row = tile * 16 + g + (i >> 1) * 8;
                if (n < batch) {
                    const size_t oi = (size_t)n * rows + row;
                    const float y = scaled ? acc[j][i] * scratch[n] : acc[j][i];
                    if (out_dtype == SANIC_BF16) ((uint16_t*)segs.out[0])[oi] = f32_to_bf16_bits(y);
                    else ((float*)segs.out[0])[oi] = y;
                }
            }
    }
}

// int4-g64 silu(gate) * up at K <= 2048: a TEAM of four warps per dual tile (16 rows of each matrix), a quarter of the K axis
// each. The layers' matrices have too few tiles for a warp per tile (512 dual tiles for 8192 rows) and too little work per tile
// for a block per tile; with four warps per tile every resident warp has one tile's quarter, all of its loads in flight at
// once (GPW groups x 2 matrices x 2 rows of 8 bytes). The three other warps hand their sums to the first through shared
// memory at a barrier of the four; it adds them in a fixed order, scales, applies silu * up and stores.
__device__ __forceinline__ void team_sync(int team) {      // the four warps of a team; a barrier of its own per team
    if (team == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
    else asm volatile("bar.sync 2, 128;" ::: "memory");
}
template <bool NORM, int NT, int GPW>
__global__ void __launch_bounds__(GW * 32, 2) gemv_w4_dual_team_kernel(const uint16_t* __restrict__ x, int batch, int K, SegTable segs, int out_dtype,
                                                                      Fused fz, int tiles) {
    extern __shared__ __align__(16) unsigned char wr_smem[];
    float* scratch = (float*)wr_smem;
    const int G = K / 64, xpitch = K * 2 + 16;
    float2* gsum = (float2*)(wr_smem + 1024);
    unsigned char* xs = wr_smem + 1024 + G * NT * 32;
    float4* comb = (float4*)(xs + 8 * NT * xpitch);       // [2 teams][3 warps][32 lanes][2 * NT]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    griddep_launch();
    griddep_wait();
    if (NORM) row_norms<false>(fz, batch, K, scratch);
    else if (fz.ds_partial) defer_scales<false>(fz, batch, scratch);
    for (int i = tid; i < batch * (K / 16); i += GW * 32) {
        const int n = i / (K / 16), c = i % (K / 16);
        const uint16_t* xr = NORM ? nullptr : x + (size_t)n * K;
        const float* xf = NORM ? fz.norm_x + (size_t)n * K : nullptr;
        const uint4 xa = load_x8<NORM, false>(xr, xf, fz.norm_gamma, NORM ? scratch[n] : 1.0f, c * 16, true);
        const uint4 xc = load_x8<NORM, false>(xr, xf, fz.norm_gamma, NORM ? scratch[n] : 1.0f, c * 16 + 8, true);
        uint4* dst = (uint4*)(xs + (size_t)n * xpitch + c * 32);
        dst[0] = make_uint4(prmt(xa.x, xa.z, 0x5410), prmt(xa.x, xa.z, 0x7632), prmt(xa.y, xa.w, 0x5410), prmt(xa.y, xa.w, 0x7632));
        dst[1] = make_uint4(prmt(xc.x, xc.z, 0x5410), prmt(xc.x, xc.z, 0x7632), prmt(xc.y, xc.w, 0x5410), prmt(xc.y, xc.w, 0x7632));
    }
    __syncthreads();
    bool xok[NT];
    const unsigned char* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = 8 * j + g < batch;
        xrow[j] = xs + (size_t)(xok[j] ? 8 * j + g : 0) * xpitch + t * 32;
    }
    auto x_frags = [&](int u, int j, uint32_t (&b)[8]) {
        const uint4 lo = xok[j] ? *(const uint4*)(xrow[j] + (size_t)u * 128) : make_uint4(0, 0, 0, 0);
        const uint4 hi = xok[j] ? *(const uint4*)(xrow[j] + (size_t)u * 128 + 16) : make_uint4(0, 0, 0, 0);
        b[0] = lo.x; b[1] = lo.y; b[2] = lo.z; b[3] = lo.w; b[4] = hi.x; b[5] = hi.y; b[6] = hi.z; b[7] = hi.w;
    };
    {
        const uint32_t ONES = 0x3F803F80u;
        for (int u = warp; u < G; u += GW) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint32_t b[8];
                x_frags(u, j, b);
                float c1[4] = {0, 0, 0, 0};
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[0], b[1]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[2], b[3]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[4], b[5]);
                mma_bf16_16816(c1, ONES, ONES, ONES, ONES, b[6], b[7]);
                if (g == 0) gsum[(u * NT + j) * 4 + t] = make_float2(c1[0], c1[1]);
            }
        }
    }
    __syncthreads();
    const int rows = segs.rows[0];
    const bool scaled = !NORM && fz.ds_partial != nullptr;
    const int team = warp >> 2, sub = warp & 3, g0 = sub * GPW;
    for (int tile = blockIdx.x * 2 + team; tile < tiles; tile += gridDim.x * 2) {
        // every load of this warp's quarter of the tile: GPW groups of rows g and g+8 of both matrices, and their scales
        uint2 wv[2][2][GPW];
        uint32_t sv[2][2][GPW / 2];
#pragma unroll
        for (int mI = 0; mI < 2; ++mI) {
            const uint8_t* Wm = (const uint8_t*)segs.w[mI];
            const uint16_t* Sm = segs.scales[mI];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const size_t wrow = (size_t)(tile * 16 + g + 8 * r);
#pragma unroll
                for (int u = 0; u < GPW; ++u) wv[mI][r][u] = ldg_stream8(Wm + wrow * (K / 2) + (size_t)(g0 + u) * 32 + t * 8);
#pragma unroll
                for (int u = 0; u < GPW / 2; ++u) sv[mI][r][u] = __ldg((const uint32_t*)(Sm + wrow * G + g0) + u);
            }
        }
        float acc[2][NT][4];
#pragma unroll
        for (int mI = 0; mI < 2; ++mI)
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[mI][j][0] = acc[mI][j][1] = acc[mI][j][2] = acc[mI][j][3] = 0.0f;
#pragma unroll
        for (int u = 0; u < GPW; ++u) {
            uint32_t b[NT][8];
            float2 cs[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) { x_frags(g0 + u, j, b[j]); cs[j] = gsum[((g0 + u) * NT + j) * 4 + t]; }
#pragma unroll
            for (int mI = 0; mI < 2; ++mI) {
                const uint32_t a0 = wv[mI][0][u].x, a1 = wv[mI][0][u].y, c0 = wv[mI][1][u].x, c1w = wv[mI][1][u].y;
                const uint32_t s0w = sv[mI][0][u >> 1], s1w = sv[mI][1][u >> 1];
                const float sc0 = (u & 1) ? bf16hi(s0w) : bf16lo(s0w), sc1 = (u & 1) ? bf16hi(s1w) : bf16lo(s1w);
                const uint32_t f0 = nib_pair(a0), f1 = nib_pair(c0), f2 = nib_pair(a0 >> 4), f3 = nib_pair(c0 >> 4);
                const uint32_t f4 = nib_pair(a0 >> 8), f5 = nib_pair(c0 >> 8), f6 = nib_pair(a0 >> 12), f7 = nib_pair(c0 >> 12);
                const uint32_t h0 = nib_pair(a1), h1 = nib_pair(c1w), h2 = nib_pair(a1 >> 4), h3 = nib_pair(c1w >> 4);
                const uint32_t h4 = nib_pair(a1 >> 8), h5 = nib_pair(c1w >> 8), h6 = nib_pair(a1 >> 12), h7 = nib_pair(c1w >> 12);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    float c[4] = {0, 0, 0, 0};
                    mma_bf16_16816(c, f0, f1, f2, f3, b[j][0], b[j][1]);
                    mma_bf16_16816(c, f4, f5, f6, f7, b[j][2], b[j][3]);
                    mma_bf16_16816(c, h0, h1, h2, h3, b[j][4], b[j][5]);
                    mma_bf16_16816(c, h4, h5, h6, h7, b[j][6], b[j][7]);
                    acc[mI][j][0] = fmaf(sc0, fmaf(-136.0f, cs[j].x, c[0]), acc[mI][j][0]);
                    acc[mI][j][1] = fmaf(sc0, fmaf(-136.0f, cs[j].y, c[1]), acc[mI][j][1]);
                    acc[mI][j][2] = fmaf(sc1, fmaf(-136.0f, cs[j].x, c[2]), acc[mI][j][2]);
                    acc[mI][j][3] = fmaf(sc1, fmaf(-136.0f, cs[j].y, c[3]), acc[mI][j][3]);
                }
            }
        }
        // the other three warps' sums to the first, in the order of their K quarters
        float4* mine = comb + ((size_t)(team * 3 + (sub - 1)) * 32 + lane) * (2 * NT);
        if (sub != 0) {
#pragma unroll
            for (int mI = 0; mI < 2; ++mI)
#pragma unroll
                for (int j = 0; j < NT; ++j) mine[mI * NT + j] = make_float4(acc[mI][j][0], acc[mI][j][1], acc[mI][j][2], acc[mI][j][3]);
        }
        team_sync(team);
        if (sub == 0) {
#pragma unroll
            for (int w = 0; w < 3; ++w) {
                const float4* theirs = comb + ((size_t)(team * 3 + w) * 32 + lane) * (2 * NT);
#pragma unroll
                for (int mI = 0; mI < 2; ++mI)
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const float4 o = theirs[mI * NT + j];
                        acc[mI][j][0] += o.x; acc[mI][j][1] += o.y; acc[mI][j][2] += o.z; acc[mI][j][3] += o.w;
                    }
            }
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = 8 * j + 2 * t + (i & 1), row = tile * 16 + g + (i >> 1) * 8;
                    if (n < batch) {
                        const float sc = scaled ? scratch[n] : 1.0f;
                        const float ga = acc[0][j][i] * sc, up = acc[1][j][i] * sc;
                        const float sig = 1.0f / (1.0f + expf(-ga));       // silu(a) * b = (a * 1/(1+exp(-a))) * b  (reference src/ir.rs:1500-1509)
                        const float y = (ga * sig) * up;
                        const size_t oi = (size_t)n * rows + row;
                        if (out_dtype == SANIC_BF16) ((uint16_t*)segs.out[0])[oi] = f32_to_bf16_bits(y);
                        else ((float*)segs.out[0])[oi] = y;
                    }
                }
        }
        team_sync(team);      // the hand-over places are free again
    }
}

template <bool W4, int NT, bool DUAL, bool NORM>
int32_t launch(sanic_ctx* ctx, const sanic_gemv_params& p, const SegTable& segs, const Fused& fz, int tiles, cudaStream_t st) {
    // Few row tiles cannot fill 148 SMs: split K over a cluster of KS CTAs per tile (each warp keeps
    // at least one 64-block of K).
    if (W4 && !DUAL && rows_form_applies(ctx, p)) {
        const size_t smem = 1024 + (size_t)(p.K / 64) * NT * 32 + (size_t)8 * NT * (p.K * 2 + 16);
        auto kern = gemv_w4_rows_kernel<NORM, NT>;
        SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const int blocks = std::min((tiles + GW - 1) / GW, 2 * ctx->sm_count);
        cudaError_t e = launch_pdl(kern, dim3(blocks), dim3(GW * 32), smem, st, (const uint16_t*)p.x, p.batch, p.K, segs, p.out_dtype, fz, tiles);
        if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemv (int4 rows): ") + cudaGetErrorString(e));
        return SANIC_OK;
    }
    // (at batch > 8 the contraction is bound by instruction issue in either form: 13.5 us against the ring-fed kernel's 14.2 stand-alone,
    // and slower inside a step, where the ring-fed kernel's start overlaps its predecessor's end; so only up to batch 8)
    if (W4 && DUAL && NT == 1 && (p.K == 2048 || p.K == 1024) && p.rows[0] % 16 == 0 && tiles >= ctx->sm_count &&
        !(getenv("SANIC_GEMV_W4_ROWS") && getenv("SANIC_GEMV_W4_ROWS")[0] == '0')) {
        const size_t smem = 1024 + (size_t)(p.K / 64) * NT * 32 + (size_t)8 * NT * (p.K * 2 + 16) + (size_t)2 * 3 * 32 * 2 * NT * sizeof(float4);
        const int blocks = std::min((tiles + 1) / 2, 2 * ctx->sm_count);
        cudaError_t e;
        if (p.K == 2048) {
            auto kern = gemv_w4_dual_team_kernel<NORM, NT, 8>;
            SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            e = launch_pdl(kern, dim3(blocks), dim3(GW * 32), smem, st, (const uint16_t*)p.x, p.batch, p.K, segs, p.out_dtype, fz, tiles);
        } else {
            auto kern = gemv_w4_dual_team_kernel<NORM, NT, 4>;
            SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            e = launch_pdl(kern, dim3(blocks), dim3(GW * 32), smem, st, (const uint16_t*)p.x, p.batch, p.K, segs, p.out_dtype, fz, tiles);
        }
        if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemv (int4 silu-mul teams): ") + cudaGetErrorString(e));
        return SANIC_OK;
    }
    int KS = 1;
    const int nblk = p.K / 64;
    // SANIC_GEMV_KS caps the split (tuning knob). Default: two CTAs per tile for a long K axis with at most one tile per SM
    // (the down projection: 2048 x 8192, four passes of loads per warp; int4 at batch 1 9.8 -> 7.1 us). The short-K
    // contractions lose with it (q/k/v with the RoPE epilogue 3.6 -> 6.9 us), and four CTAs per tile lose everywhere.
    static const int ks_env = getenv("SANIC_GEMV_KS") ? atoi(getenv("SANIC_GEMV_KS")) : 0;
    const int ks_cap = ks_env > 0 ? ks_env : ((p.K >= 4096 && tiles <= ctx->sm_count && (p.epilogue == SANIC_EPI_STORE || p.epilogue == SANIC_EPI_RESIDUAL_ADD)) ? 2 : 1);
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

bool sanic::gemv::rows_form_applies(const sanic_ctx* ctx, const sanic_gemv_params& p) {
    return p.weight_dtype == SANIC_I4 && p.n_segments == 1 && p.epilogue == SANIC_EPI_STORE && !(p.ds_partial && p.norm_x) &&
           p.K % 256 == 0 && p.K <= (p.batch > 8 ? 2048 : 4096) && p.rows[0] % 16 == 0 && p.rows[0] / 16 >= 16 * ctx->sm_count &&
           !(getenv("SANIC_GEMV_W4_ROWS") && getenv("SANIC_GEMV_W4_ROWS")[0] == '0');
}

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
    // (int4 q/k/v with the RoPE + cache epilogue: 192 tiles, measured 4.7 us register-staged against 6.3 us ring-fed)
    if (wide && ring && !p->norm_x && !rows_form_applies(ctx, *p) && !(w4 && p->epilogue == SANIC_EPI_ROPE_CACHE)) {
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
