// Body of the decode-batch contraction, shared by the stand-alone kernel (gemv.cu) and the persistent
// decode-step kernel (decode_step.cu). See gemv.cu for the design notes.
#pragma once
#include "common.cuh"

namespace sanic {
namespace gemv {

constexpr int GW = 8;  // warps per CTA

struct SegTable {
    const void* w[3];
    const uint16_t* scales[3];
    void* out[3];
    int rows[3];
    int tile_begin[4];
};
struct Fused {
    const float* norm_x; const uint16_t* norm_gamma; float norm_eps;
    const float* rope_table; const int32_t* rope_position; uint16_t* rope_q_out; uint16_t* rope_k_cache; uint16_t* rope_v_cache;
    int q_heads, kv_heads, head_dim, ctx;
    // deferred normaliser: what a residual-add epilogue also writes for the next contraction, and what a contraction's
    // outputs are scaled by (see sanic_gemv_params)
    uint16_t* nx_out; const uint16_t* nx_gamma; float* nx_partial;
    const float* ds_partial; int ds_tiles; float ds_eps;
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
__device__ __forceinline__ const void* pick3(const void* const (&a)[3], int i) { return i == 0 ? a[0] : (i == 1 ? a[1] : a[2]); }

// 8 consecutive activations of batch column n starting at k as four packed bf16x2 registers.
// L2READ: the activations may have been written by another SM earlier in the same kernel (the persistent
// decode step), so they are read from L2; a stand-alone kernel reads them through L1, where every tile
// after the first on an SM hits.
template <bool NORM, bool L2READ>
__device__ __forceinline__ uint4 load_x8(const uint16_t* xrow, const float* xf, const uint16_t* gamma, float den, int k,
                                         bool ok) {
    if (!ok) return make_uint4(0, 0, 0, 0);
    if (!NORM) return L2READ ? __ldcg((const uint4*)(xrow + k)) : __ldg((const uint4*)(xrow + k));
    float4 a = L2READ ? __ldcg((const float4*)(xf + k)) : __ldg((const float4*)(xf + k));
    float4 b = L2READ ? __ldcg((const float4*)(xf + k + 4)) : __ldg((const float4*)(xf + k + 4));
    uint4 g = __ldg((const uint4*)(gamma + k));
    uint4 r;
    // `den` holds 1/sqrt(mean(x^2)+eps): one multiply per element instead of a division
    r.x = pack_bf16x2((a.x * bf16lo(g.x)) * den, (a.y * bf16hi(g.x)) * den);
    r.y = pack_bf16x2((a.z * bf16lo(g.y)) * den, (a.w * bf16hi(g.y)) * den);
    r.z = pack_bf16x2((b.x * bf16lo(g.z)) * den, (b.y * bf16hi(g.z)) * den);
    r.w = pack_bf16x2((b.z * bf16lo(g.w)) * den, (b.w * bf16hi(g.w)) * den);
    return r;
}

// Block barrier of the tile's GW*32 threads: the CTA barrier in a stand-alone kernel; in the persistent
// step the block also holds a producer warp that never joins, so the consumers meet on a named barrier.
template <bool PERSIST>
__device__ __forceinline__ void block_sync() {
    if (PERSIST) asm volatile("bar.sync 2, 256;" ::: "memory");
    else __syncthreads();
}

// 1/sqrt(mean(x^2) + eps) of every activation row into scratch[0..batch): every warp sums its eighth of each
// row, so the norm costs one load round trip, not sixteen. All GW*32 threads of the block call this.
// L2READ is also the persistent-step form (reads through L2, consumer barrier).
template <bool L2READ>
__device__ __forceinline__ void row_norms(const Fused& fz, int batch, int K, float* scratch) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* s_den = scratch;
    float (*s_part)[GW] = reinterpret_cast<float (*)[GW]>(scratch + 16);
    const int kw = K / GW;
    for (int n = 0; n < batch; ++n) {
        const float* xr = fz.norm_x + (size_t)n * K + warp * kw;
        float ss = 0.0f;
        for (int i = lane * 4; i < kw; i += 128) {
            float4 v = L2READ ? __ldcg((const float4*)(xr + i)) : __ldg((const float4*)(xr + i));
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[n][warp] = ss;
    }
    block_sync<L2READ>();
    if (tid < batch) {
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < GW; ++w) tot += s_part[tid][w];
        s_den[tid] = 1.0f / sqrtf(tot * (1.0f / (float)K) + fz.norm_eps);
    }
    block_sync<L2READ>();
}

// 1 / sqrt(mean(x^2) + eps) of every activation row from the per-tile sums a residual-add epilogue left
// (Fused::ds_partial), into scratch[0..batch): the 16 threads of a row add tiles r, r+16, ... and meet in a fixed
// xor tree. All GW*32 threads of the block call this.
template <bool L2READ>
__device__ __forceinline__ void defer_scales(const Fused& fz, int batch, float* scratch) {
    const int tid = threadIdx.x, n = tid >> 4, r = tid & 15;
    float v = 0.0f;
    if (n < batch)
        for (int t = r; t < fz.ds_tiles; t += 16) {
            const float* p = fz.ds_partial + (size_t)n * fz.ds_tiles + t;
            v += L2READ ? __ldcg(p) : __ldg(p);
        }
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    if (n < batch && r == 0) scratch[n] = 1.0f / sqrtf(v * (1.0f / (float)(fz.ds_tiles * 16)) + fz.ds_eps);
    block_sync<L2READ>();
}

// Shared scratch one tile needs, in floats: row norms [16], their per-warp parts [16][GW], the per-warp
// accumulators [GW][NM][16][8*NT+1] and the block sum [NM][16][8*NT+1].
template <int NT, bool DUAL>
__host__ __device__ constexpr int scratch_floats() {
    return 16 + 16 * GW + (GW + 1) * (DUAL ? 2 : 1) * 16 * (8 * NT + 1);
}

// Floats of one set of per-warp partial sums; a caller that runs several tiles through one block may alternate between two
// sets (`parity`) so that a tile's epilogue and the next tile's contraction need no barrier between them.
template <int NT, bool DUAL>
__host__ __device__ constexpr int red_floats() { return GW * (DUAL ? 2 : 1) * 16 * (8 * NT + 1); }

// Second half of a tile: the GW warps' partial sums are added in a fixed order, then the epilogue runs. Without a K split
// across a cluster the threads that run the epilogue add the eight partials themselves: one block barrier per tile.
template <int NT, bool DUAL, bool PERSIST>
__device__ __forceinline__ void tile_finish(float (&acc)[DUAL ? 2 : 1][NT][4], int batch, const SegTable& segs, int out_dtype,
                                            int epilogue, const float* residual, const Fused& fz, int KS, int krank, int seg,
                                            int tile, float* scratch, bool have_res = false, float res_pre = 0.0f, int parity = 0) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int NM = DUAL ? 2 : 1, RW = 8 * NT + 1;
    float (*red)[NM][16][RW] = reinterpret_cast<float (*)[NM][16][RW]>(scratch + 16 + 16 * GW + parity * red_floats<NT, DUAL>());   // [GW][NM][16][RW]
    float (*csum)[16][RW] = reinterpret_cast<float (*)[16][RW]>(scratch + 16 + 16 * GW + GW * NM * 16 * RW);  // [NM][16][RW], K split only
    const bool rope = (epilogue == SANIC_EPI_ROPE_CACHE);
    const bool scaled = fz.ds_partial != nullptr;      // scratch[n] holds the row's deferred 1/sqrt(.)
    // deterministic cross-warp sum: red[warp][matrix][row 0..15][col 0..8*NT)
#pragma unroll
    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            red[warp][mI][g][8 * j + 2 * t] = acc[mI][j][0];
            red[warp][mI][g][8 * j + 2 * t + 1] = acc[mI][j][1];
            red[warp][mI][g + 8][8 * j + 2 * t] = acc[mI][j][2];
            red[warp][mI][g + 8][8 * j + 2 * t + 1] = acc[mI][j][3];
        }
    block_sync<PERSIST>();
    if (KS > 1) {
        // CTA sum in a fixed warp order, then the cluster's CTAs are summed in rank order by rank 0 through distributed
        // shared memory: deterministic, no global scratch.
        for (int idx = tid; idx < NM * 16 * 8 * NT; idx += GW * 32) {
            const int n = idx % (8 * NT), r = (idx / (8 * NT)) % 16, mI = idx / (8 * NT * 16);
            float sv = 0.0f;
#pragma unroll
            for (int w = 0; w < GW; ++w) sv += red[w][mI][r][n];
            csum[mI][r][n] = sv;
        }
        block_sync<PERSIST>();
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (krank == 0) {
            for (int idx = tid; idx < NM * 16 * 8 * NT; idx += GW * 32) {
                const int n = idx % (8 * NT), r = (idx / (8 * NT)) % 16, mI = idx / (8 * NT * 16);
                float sv = csum[mI][r][n];
                const uint32_t local = smem_u32(&csum[mI][r][n]);
                for (int kr = 1; kr < KS; ++kr) {
                    uint32_t remote; float v;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(kr));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
                    sv += v;
                }
                red[0][mI][r][n] = sv;     // rank 0 publishes the cluster total for its epilogue
            }
        }
        // peers stay alive until rank 0 has read their shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (krank != 0) return;
        block_sync<PERSIST>();
    }
    // the epilogue reads the cluster total rank 0 published, or, without a K split, adds the warps' partials in warp order
    auto total = [&](int mI, int r, int n) -> float {
        if (KS > 1) return red[0][mI][r][n];
        float sv = 0.0f;
#pragma unroll
        for (int w = 0; w < GW; ++w) sv += red[w][mI][r][n];
        return sv;
    };
    if (rope) {
        // thread (r < 8, n): partners a = row r (d0 = 8*sub + r) and b = row r + 8 (d0 + D/2)
        const int D = fz.head_dim, F = D / 2, tph = D / 16;
        const int head = tile / tph, sub = tile % tph;
        const int pos = *fz.rope_position;
        for (int idx = tid; idx < 8 * batch; idx += GW * 32) {
            const int n = idx / 8, r = idx % 8;
            const float sc = scaled ? scratch[n] : 1.0f;
            const float a = total(0, r, n) * sc, b = total(0, r + 8, n) * sc;
            const int d0 = 8 * sub + r;
            if (pos < 0 || pos >= fz.ctx) continue;
            if (seg < 2) {
                const float* cs = fz.rope_table + 2 * ((size_t)pos * F + d0);
                const float c = cs[0], sn = cs[1];
                const uint16_t o0 = f32_to_bf16_bits(a * c + (-b) * sn), o1 = f32_to_bf16_bits(b * c + a * sn);
                uint16_t* dst = (seg == 0) ? fz.rope_q_out + ((size_t)n * fz.q_heads + head) * D
                                           : fz.rope_k_cache + (((size_t)n * fz.kv_heads + head) * fz.ctx + pos) * D;
                dst[d0] = o0; dst[d0 + F] = o1;
            } else {
                uint16_t* dst = fz.rope_v_cache + ((size_t)n * fz.kv_heads + head) * D * (size_t)fz.ctx;
                dst[(size_t)d0 * fz.ctx + pos] = f32_to_bf16_bits(a);
                dst[(size_t)(d0 + F) * fz.ctx + pos] = f32_to_bf16_bits(b);
            }
        }
        return;
    }
    const int row0 = tile * 16;
    const int rows = seg == 0 ? segs.rows[0] : (seg == 1 ? segs.rows[1] : segs.rows[2]);
    void* outp = seg == 0 ? segs.out[0] : (seg == 1 ? segs.out[1] : segs.out[2]);
    for (int idx = tid; idx < 16 * batch; idx += GW * 32) {
        int n = idx / 16, r = idx % 16;  // consecutive threads -> consecutive rows (contiguous in out[n][row])
        const float sc = scaled ? scratch[n] : 1.0f;
        float y = total(0, r, n) * sc;
        if (DUAL) {  // silu(a) * b = (a * 1/(1+exp(-a))) * b  (reference src/ir.rs:1500-1509)
            const float ga = y, up = total(NM - 1, r, n) * sc;
            float sig = 1.0f / (1.0f + expf(-ga));
            y = (ga * sig) * up;
        }
        size_t oi = (size_t)n * rows + row0 + r;
        // `res_pre` is this thread's residual value when the caller loaded it ahead of the contraction (idx == tid then)
        if (epilogue == SANIC_EPI_RESIDUAL_ADD) y = ((have_res && idx == tid) ? res_pre : (PERSIST ? __ldcg(residual + oi) : residual[oi])) + y;
        if (out_dtype == SANIC_BF16) ((uint16_t*)outp)[oi] = f32_to_bf16_bits(y);
        else ((float*)outp)[oi] = y;
        if (epilogue == SANIC_EPI_RESIDUAL_ADD && fz.nx_out) {
            // the next contraction's activations and this tile's share of sum y^2: the 16 threads of a batch row are 16
            // neighbouring lanes (16 * batch is a multiple of 16, so the active lanes are whole groups)
            fz.nx_out[oi] = f32_to_bf16_bits(y * bf16_to_f32(fz.nx_gamma[row0 + r]));
            // lanes of this warp inside the loop: all 32, or the lower 16 when 16 * batch ends in the middle of the warp
            const unsigned live = (16 * batch - (int)(threadIdx.x & ~31u) >= 32) ? 0xffffffffu : 0x0000ffffu;
            float sq = y * y;
            sq += __shfl_xor_sync(live, sq, 8);
            sq += __shfl_xor_sync(live, sq, 4);
            sq += __shfl_xor_sync(live, sq, 2);
            sq += __shfl_xor_sync(live, sq, 1);
            if (r == 0) fz.nx_partial[(size_t)n * (rows / 16) + tile] = sq;
        }
    }
}

// One row tile of the contraction. `block` is the linear block index (tile * KS + K-rank); `pdl` says
// whether the caller is a stand-alone kernel that must order itself after its stream predecessor.
// PERSIST is the form the persistent decode step calls: activations (and the residual) are read from L2
// and the row norms are already in scratch[0..batch), computed once per phase by the caller.
template <bool W4, int NT, bool DUAL, bool NORM, bool PERSIST = false>
__device__ __forceinline__ void gemv_tile(const uint16_t* __restrict__ x, int batch, int K, const SegTable& segs,
                                          int n_segments, int out_dtype, int epilogue, const float* residual,
                                          const Fused& fz, int KS, int block, bool pdl, float* scratch) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // carve the caller's shared scratch (scratch_floats<NT, DUAL>() floats)
    float* s_den = scratch;                                                                                  // [16]
    const int g = lane >> 2, t = lane & 3;
    // KS CTAs of one thread-block cluster share a row tile and split K between them
    const int gtile = block / KS, krank = block % KS;
    int seg = 0;
    if (!DUAL) {
        if (n_segments > 1 && gtile >= segs.tile_begin[1]) seg = 1;
        if (n_segments > 2 && gtile >= segs.tile_begin[2]) seg = 2;
    }
    const int tile = gtile - (seg == 0 ? segs.tile_begin[0] : (seg == 1 ? segs.tile_begin[1] : segs.tile_begin[2]));
    const bool rope = (epilogue == SANIC_EPI_ROPE_CACHE);
    // weight rows of A-fragment rows g and g+8
    int wrow0, wrow1;
    if (rope) {   // rotate-half partners of one head: d = 8*sub + g and d + D/2
        const int tph = fz.head_dim / 16, head = tile / tph, sub = tile % tph;
        wrow0 = head * fz.head_dim + 8 * sub + g;
        wrow1 = wrow0 + fz.head_dim / 2;
    } else {
        wrow0 = tile * 16 + g;
        wrow1 = wrow0 + 8;
    }
    constexpr int NM = DUAL ? 2 : 1;
    const int nblk = K / 64;
    const int cb0 = (krank * nblk) / KS, cb1 = ((krank + 1) * nblk) / KS;   // this CTA's K range, in 64-blocks
    const int b0 = cb0 + (warp * (cb1 - cb0)) / GW, b1 = cb0 + ((warp + 1) * (cb1 - cb0)) / GW;

    // Weights do not depend on the previous kernel of the step: ask L2 for this warp's whole weight
    // slice (16 rows x its K range) before waiting for that kernel, so HBM keeps streaming while
    // the predecessor drains.
    {
        const size_t row_bytes = W4 ? (size_t)K / 2 : (size_t)K * 2;
        const int blk_bytes = W4 ? 32 : 128;
        const int span = (b1 - b0) * blk_bytes;
        const int lines = (span + 127) / 128;
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            const char* wbase = (const char*)pick3(segs.w, DUAL ? mI : seg);
            for (int i = lane; i < 16 * lines; i += 32) {
                const int r = i / lines, ln = i % lines;
                const size_t wrow = (r < 8) ? (size_t)(wrow0 - g + r) : (size_t)(wrow1 - g + r - 8);
                asm volatile("prefetch.global.L2 [%0];" ::"l"(wbase + wrow * row_bytes + (size_t)b0 * blk_bytes + (size_t)ln * 128));
            }
        }
    }
    if (pdl) { griddep_launch(); griddep_wait(); }

    if (NORM && !PERSIST) row_norms<false>(fz, batch, K, scratch);
    if (!NORM && !PERSIST && fz.ds_partial) defer_scales<false>(fz, batch, scratch);

    float acc[NM][NT][4];
#pragma unroll
    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[mI][j][0] = acc[mI][j][1] = acc[mI][j][2] = acc[mI][j][3] = 0.0f;

    const uint16_t* xrow[NT];
    const float* xf[NT];
    float den[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = (8 * j + g) < batch;
        const int n = xok[j] ? (8 * j + g) : 0;
        xrow[j] = x + (size_t)n * K;
        xf[j] = NORM ? fz.norm_x + (size_t)n * K : nullptr;
        den[j] = NORM ? s_den[n] : 1.0f;
    }
    const uint16_t* gam = fz.norm_gamma;

    if (!W4) {
        const uint16_t* wr[NM][2];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            const uint16_t* W = (const uint16_t*)pick3(segs.w, DUAL ? mI : seg);
            wr[mI][0] = W + (size_t)wrow0 * K;
            wr[mI][1] = W + (size_t)wrow1 * K;
        }
        constexpr int U = (DUAL || NT == 2) ? 2 : 4;     // 64-blocks in flight per warp: what 128 registers hold without spilling
        for (int blk = b0; blk < b1; blk += U) {
            const int nb = min(U, b1 - blk);      // uniform across the warp
            uint4 a[U][NM][2][2];
            uint4 xb[U][NT][2];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < nb) {
                    int kb = (blk + u) * 64;
#pragma unroll
                    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            // k permutation: thread t owns 16 consecutive k of the 64-block (two 16-byte loads side by side),
                            // so the four threads of a row read one whole 128-byte line; the activations use the same one
                            a[u][mI][r][0] = ldg_stream16(wr[mI][r] + kb + t * 16);
                            a[u][mI][r][1] = ldg_stream16(wr[mI][r] + kb + t * 16 + 8);
                        }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < nb) {
                    int kb = (blk + u) * 64;
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        xb[u][j][0] = load_x8<NORM, PERSIST>(xrow[j], xf[j], gam, den[j], kb + t * 16, xok[j]);
                        xb[u][j][1] = load_x8<NORM, PERSIST>(xrow[j], xf[j], gam, den[j], kb + t * 16 + 8, xok[j]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < nb) {
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
            }
        }
    } else {
        const int G = K / 64;  // groups per row
        const uint8_t* wr[NM][2];
        const uint16_t* sr[NM][2];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI) {
            const uint8_t* W = (const uint8_t*)pick3(segs.w, DUAL ? mI : seg);
            const int si = DUAL ? mI : seg;
            const uint16_t* S = si == 0 ? segs.scales[0] : (si == 1 ? segs.scales[1] : segs.scales[2]);
            wr[mI][0] = W + (size_t)wrow0 * (K / 2);
            wr[mI][1] = W + (size_t)wrow1 * (K / 2);
            sr[mI][0] = S + (size_t)wrow0 * G;
            sr[mI][1] = S + (size_t)wrow1 * G;
        }
        constexpr int U = DUAL ? 2 : 4;
        const uint32_t ONES = 0x3F803F80u;
        auto do_group = [&](const uint2 (&wv)[NM][2], const float (&sc)[NM][2], int blk) {
            int kb = blk * 64 + t * 16;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                uint4 xa = load_x8<NORM, PERSIST>(xrow[j], xf[j], gam, den[j], kb, xok[j]);
                uint4 xc = load_x8<NORM, PERSIST>(xrow[j], xf[j], gam, den[j], kb + 8, xok[j]);
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
        for (int blk = b0; blk < b1; blk += U) {
            const int nb = min(U, b1 - blk);
            uint2 wv[U][NM][2];
            float sc[U][NM][2];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < nb) {
#pragma unroll
                    for (int mI = 0; mI < NM; ++mI)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            wv[u][mI][r] = ldg_stream8(wr[mI][r] + (size_t)(blk + u) * 32 + t * 8);
                            sc[u][mI][r] = bf16_to_f32(__ldg(sr[mI][r] + blk + u));
                        }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (u < nb) do_group(wv[u], sc[u], blk + u);
        }
    }

    tile_finish<NT, DUAL, PERSIST>(acc, batch, segs, out_dtype, epilogue, residual, fz, KS, krank, seg, tile, scratch);
}

// Host side: validate one contraction and build the kernel's segment table. `tiles` is the number of
// 16-row tiles (one thread block each, before any K split).
inline int32_t host_prepare(sanic_ctx* ctx, const sanic_gemv_params* p, SegTable& segs, Fused& fz, int& tiles) {
    SANIC_REQUIRE(ctx, (p->x || p->norm_x) && p->batch >= 1 && p->batch <= 16, "gemv: batch must be in [1, 16]");
    SANIC_REQUIRE(ctx, p->K >= 64 && p->K % 64 == 0, "gemv: K must be a multiple of 64");
    SANIC_REQUIRE(ctx, p->n_segments >= 1 && p->n_segments <= 3, "gemv: 1..3 weight segments");
    if (p->weight_dtype != SANIC_BF16 && p->weight_dtype != SANIC_I4)
        return sanic_fail(ctx, SANIC_ERR_DTYPE, "gemv: weights must be bf16 or int4");
    SANIC_REQUIRE(ctx, p->weight_dtype != SANIC_I4 || p->group == 64, "gemv: int4 group size must be 64");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_F32 || p->out_dtype == SANIC_BF16, "gemv: output must be f32 or bf16");
    SANIC_REQUIRE(ctx, ((uintptr_t)p->x % 16) == 0 && ((uintptr_t)p->norm_x % 16) == 0 && ((uintptr_t)p->norm_gamma % 16) == 0,
                  "gemv: activations must be 16-byte aligned");
    SANIC_REQUIRE(ctx, !p->norm_x || p->norm_gamma, "gemv: an inlined norm needs its weight");
    const bool dual = p->epilogue == SANIC_EPI_SILU_MUL;
    const bool rope = p->epilogue == SANIC_EPI_ROPE_CACHE;
    SANIC_REQUIRE(ctx, !dual || (p->n_segments == 2 && p->rows[0] == p->rows[1]), "gemv: silu-mul needs two equal segments");
    SANIC_REQUIRE(ctx, p->epilogue != SANIC_EPI_RESIDUAL_ADD || (p->residual && p->n_segments == 1),
                  "gemv: residual-add needs one segment and a residual");
    if (rope) {
        SANIC_REQUIRE(ctx, p->n_segments == 3 && p->rope_table && p->rope_position && p->rope_q_out && p->rope_k_cache &&
                      p->rope_v_cache, "gemv: the rope-cache epilogue needs q, k, v segments and its buffers");
        SANIC_REQUIRE(ctx, (p->rope_head_dim == 64 || p->rope_head_dim == 128) && p->rope_ctx > 0 &&
                      p->rows[0] == p->rope_q_heads * p->rope_head_dim && p->rows[1] == p->rope_kv_heads * p->rope_head_dim &&
                      p->rows[2] == p->rows[1], "gemv: rope-cache segment rows must be heads * head_dim");
    }
    segs = SegTable{};
    tiles = 0;
    for (int i = 0; i < p->n_segments; ++i) {
        SANIC_REQUIRE(ctx, p->w[i] && p->rows[i] > 0 && p->rows[i] % 16 == 0,
                      "gemv: segment rows must be a positive multiple of 16");
        SANIC_REQUIRE(ctx, p->out[i] || (dual && i == 1) || rope, "gemv: null output");
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
    fz = Fused{p->norm_x, (const uint16_t*)p->norm_gamma, p->norm_eps, p->rope_table, p->rope_position,
               (uint16_t*)p->rope_q_out, (uint16_t*)p->rope_k_cache, (uint16_t*)p->rope_v_cache,
               p->rope_q_heads, p->rope_kv_heads, p->rope_head_dim, p->rope_ctx,
               (uint16_t*)p->nx_out, (const uint16_t*)p->nx_gamma, p->nx_partial, p->ds_partial, p->ds_tiles, p->ds_eps};
    const bool nx = p->nx_out || p->nx_gamma || p->nx_partial;
    SANIC_REQUIRE(ctx, !nx || (p->nx_out && p->nx_gamma && p->nx_partial && p->epilogue == SANIC_EPI_RESIDUAL_ADD && p->out_dtype == SANIC_F32),
                  "gemv: the deferred-norm outputs need all three buffers, the residual-add epilogue and an f32 output");
    SANIC_REQUIRE(ctx, !p->ds_partial || (!p->norm_x && p->ds_tiles * 16 == p->K && p->ds_eps >= 0.0f),
                  "gemv: a deferred scale needs ds_tiles = K / 16 and no inlined norm");
    return SANIC_OK;
}

}  // namespace gemv
}  // namespace sanic
