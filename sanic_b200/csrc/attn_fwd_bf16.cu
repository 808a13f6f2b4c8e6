// Online-softmax fold for prefill (FlashAttention forward), bf16 storage, head_dim 64, on the
// 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05 MMAs with TMEM accumulators,
// Q/K/V tiles arrive by TMA, and the (m, l, o) carrier of each query row is kept by the thread that
// owns that row (one TMEM lane per row, so row max and row sum need no shuffles).
//
// One CTA folds 256 query rows of one (batch, query head) as two 128-row tiles that ping-pong on
// the tensor core: while one tile's softmax warpgroup turns S into P, the other tile's MMAs run.
//   warp 0       TMA producer: Q once, then K_j / V_j tiles of 128 keys through a 5-stage ring
//   warp 1       MMA issuer: per key tile  PV(0,j) QK(0,j+1) PV(1,j) QK(1,j+1)
//   warp 2       TMEM allocator (S0 S1 | P0 P1 | O0 O1 = 2x128 + 2x64 + 2x64 columns, all 512)
//   warps 4-7    softmax + correction + epilogue of tile 0
//   warps 8-11   the same for tile 1
// P never touches shared memory: the softmax threads write bf16 pairs back to tensor memory and
// the PV MMA takes its A operand from there.
// Masks: causal (key > row), sliding window (key < row - window + 1) and the ragged key tail are
// applied only in tiles that straddle an edge; tiles wholly outside the visible range are never
// loaded (a prefix-masked fold may stop at the mask edge: it contributes exact zeros).
// The rescale of O by exp(m_old - m_new) is skipped when no row of the warp moved its max.
// Every mbarrier wait is bounded and reports through the context's status word.
//
// Roofline: tensor-bound, 4*B*Hq*S^2*D/2 FLOP for causal; the exponentials (one per score) run on
// the 16-per-clock SFU and bound the tensor pipe to about half of its peak at head_dim 64.
#include "tc_common.cuh"

namespace {
using namespace sanic;
using namespace sanic::tc;

constexpr int D = 64, BM = 128, BN = 128, KV_STAGES = 5;
// tensor-memory columns: S0 S1 (f32 scores), P0 P1 (bf16 probabilities, two per column), O0 O1 (f32 outputs)
constexpr int TM_S = 0, TM_P = 256, TM_O = 384;
constexpr int Q_BYTES = BM * D * 2;        // 16 KB per query tile
constexpr int KV_BYTES = BN * D * 2;       // 16 KB per K or V tile
constexpr int NTHREADS = 384;

struct FShared {
    uint64_t q_full[2], q_empty[2];                                   // query tiles, double-buffered across work items
    uint64_t k_full[KV_STAGES], v_full[KV_STAGES], kv_empty[KV_STAGES];
    uint64_t s_full[2], s_free[2], p_full[2], pv_done[2], o_free[2];   // per query tile
    uint32_t tmem_base;
    volatile int abort_flag;
};

struct FParams {
    void* out;
    int batch, q_heads, kv_heads, q_len, kv_len, causal, window;
    float scale;
    int n_mb, n_items;      // 256-row query blocks per (batch, head); work items = n_mb * q_heads * batch
};

// One work item = 256 query rows of one (batch, query head): two 128-row tiles and the key tiles they see.
struct Item {
    int m0, h, b, hk;
    int jb[2], je[2], j_begin, j_end;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed pairs: one instruction for two adjacent columns.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1) {   // d += a
    asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}

// key-tile range [jb, je) that tile rows [r0, r0+127] can see
__device__ __forceinline__ void tile_range(const FParams& p, int r0, int nkv, int& jb, int& je) {
    jb = 0; je = nkv;
    if (r0 >= p.q_len) { jb = je = 0; return; }
    int rmax = min(r0 + BM - 1, p.q_len - 1);
    if (p.causal || p.window > 0) je = min(nkv, rmax / BN + 1);
    if (p.window > 0) jb = max(0, r0 - p.window + 1) / BN;
}

// Item index of this CTA's n-th round: rounds alternate direction over the CTAs so that the CTA that got
// the heaviest item of one round gets the lightest of the next.
__device__ __forceinline__ int item_of_round(int n) {
    const int G = gridDim.x, c = blockIdx.x;
    return n * G + ((n & 1) ? G - 1 - c : c);
}

// Items are ordered heaviest first (latest query block first; within a block the query heads of one
// key/value head are adjacent so concurrent CTAs share K/V tiles in L2).
__device__ __forceinline__ Item make_item(const FParams& p, int k, int nkv) {
    Item it;
    const int per_mb = p.q_heads * p.batch;
    const int mb = p.n_mb - 1 - k / per_mb, rem = k % per_mb;
    it.h = rem % p.q_heads; it.b = rem / p.q_heads;
    it.hk = it.h / (p.q_heads / p.kv_heads);
    it.m0 = mb * 2 * BM;
    tile_range(p, it.m0, nkv, it.jb[0], it.je[0]);
    tile_range(p, it.m0 + BM, nkv, it.jb[1], it.je[1]);
    const bool act1 = it.je[1] > it.jb[1];
    it.j_begin = act1 ? min(it.jb[0], it.jb[1]) : it.jb[0];
    it.j_end = act1 ? max(it.je[0], it.je[1]) : it.je[0];
    return it;
}

__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, FParams p, int* err) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* aligned = smem_dyn + (base - raw);
    const uint32_t q_addr = base, kv_addr = base + 4 * Q_BYTES;
    FShared* sh = (FShared*)(aligned + 4 * Q_BYTES + KV_STAGES * 2 * KV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkv = (p.kv_len + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->q_full[i], 1); mbar_init(&sh->q_empty[i], 1); }
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&sh->k_full[s], 1); mbar_init(&sh->v_full[s], 1); mbar_init(&sh->kv_empty[s], 1); }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&sh->s_full[t], 1); mbar_init(&sh->s_free[t], 4); mbar_init(&sh->p_full[t], 4);
            mbar_init(&sh->pv_done[t], 1); mbar_init(&sh->o_free[t], 4);
        }
        sh->abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 2) tmem_alloc(&sh->tmem_base, 512);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = sh->tmem_base;
    volatile int* abortp = &sh->abort_flag;

    // Every role walks the same item sequence: its own sub-list; all barrier
    // parities come from running counts, so nothing is re-initialised between items.
    if (warp == 0) {
        if (lane == 0) {
            int stage = 0; uint32_t phase = 1;
            bool ok = true;
            int n = 0;
            for (int k = item_of_round(0); k < p.n_items && ok; k = item_of_round(++n)) {
                const Item w = make_item(p, k, nkv);
                const int qb = n & 1;
                ok = mbar_wait(&sh->q_empty[qb], ((n >> 1) & 1) ^ 1, abortp, err, 10);
                if (!ok) break;
                const int qrow = (w.b * p.q_heads + w.h) * p.q_len + w.m0;
                mbar_expect_tx(&sh->q_full[qb], 2 * Q_BYTES);
                tma_load_2d(q_addr + qb * 2 * Q_BYTES, &map_q, &sh->q_full[qb], 0, qrow);
                tma_load_2d(q_addr + qb * 2 * Q_BYTES + Q_BYTES, &map_q, &sh->q_full[qb], 0, qrow + BM);
                const int krow = (w.b * p.kv_heads + w.hk) * p.kv_len;
                for (int j = w.j_begin; j < w.j_end; ++j) {
                    ok = mbar_wait(&sh->kv_empty[stage], phase, abortp, err, 11);
                    if (!ok) break;
                    const uint32_t ka = kv_addr + stage * 2 * KV_BYTES;
                    mbar_expect_tx(&sh->k_full[stage], KV_BYTES);
                    tma_load_2d(ka, &map_k, &sh->k_full[stage], 0, krow + j * BN);
                    mbar_expect_tx(&sh->v_full[stage], KV_BYTES);
                    tma_load_2d(ka + KV_BYTES, &map_v, &sh->v_full[stage], 0, krow + j * BN);
                    if (++stage == KV_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(BM, BN, false);
            constexpr uint32_t idesc_pv = make_idesc(BM, D, true);
            // The two tiles advance independently. QK(t, j+1) is issued as soon as tile t's softmax
            // warps have pulled S(t, j) into registers, so the next scores are ready before the
            // exponentials of the current ones finish; PV(t, j) follows when P(t, j) is written.
            // This thread serves the four events (S free / P full, per tile) in arrival order.
            bool ok = true;
            int n = 0;
            uint32_t u_base = 0;                 // key tiles of all earlier items: position in the K/V ring
            uint32_t n_qk[2] = {0, 0}, n_pv[2] = {0, 0};   // QK / PV issues so far per tile, over all items
            uint32_t n_act[2] = {0, 0};          // earlier items in which the tile had work (its O was read back)
            for (int k = item_of_round(0); k < p.n_items && ok; k = item_of_round(++n)) {
                const Item w = make_item(p, k, nkv);
                const int qb = n & 1;
                ok = mbar_wait(&sh->q_full[qb], (n >> 1) & 1, abortp, err, 12);
                if (!ok) break;
                fence_after();
                int jq[2] = {w.jb[0], w.jb[1]};      // next key tile whose QK is to be issued
                int jp[2] = {w.jb[0], w.jb[1]};      // next key tile whose PV is to be issued
                int jr = w.j_begin;                  // next ring slot to hand back to the producer
                bool q_released = false;
                uint32_t idle = 0;
                while (ok && (jp[0] < w.je[0] || jp[1] < w.je[1])) {
                    bool progressed = false;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (jq[t] < w.je[t]) {
                            const uint32_t u = u_base + (uint32_t)(jq[t] - w.j_begin);
                            const int stage = u % KV_STAGES;
                            if ((n_qk[t] == 0 || mbar_test(&sh->s_free[t], (n_qk[t] - 1) & 1)) &&
                                mbar_test(&sh->k_full[stage], (u / KV_STAGES) & 1)) {
                                fence_after();
                                const uint64_t ad = make_desc(q_addr + (qb * 2 + t) * Q_BYTES, 16, 1024);
                                const uint64_t bd = make_desc(kv_addr + stage * 2 * KV_BYTES, 16, 1024);
#pragma unroll
                                for (int kk = 0; kk < D / 16; ++kk) umma_f16(tmem + TM_S + t * BN, ad + 2 * kk, bd + 2 * kk, idesc_qk, kk > 0 ? 1u : 0u);
                                umma_commit(&sh->s_full[t]);
                                jq[t]++; n_qk[t]++; progressed = true;
                            }
                        }
                        if (jp[t] < jq[t]) {
                            const uint32_t u = u_base + (uint32_t)(jp[t] - w.j_begin);
                            const int stage = u % KV_STAGES;
                            const bool first = (jp[t] == w.jb[t]);
                            // the first PV of an item overwrites O_t: the epilogue of the tile's previous item must have read it
                            if (mbar_test(&sh->p_full[t], n_pv[t] & 1) && mbar_test(&sh->v_full[stage], (u / KV_STAGES) & 1) &&
                                (!first || n_act[t] == 0 || mbar_test(&sh->o_free[t], (n_act[t] - 1) & 1))) {
                                fence_after();
                                const uint64_t vd = make_desc(kv_addr + stage * 2 * KV_BYTES + KV_BYTES, 1024, 1024);
#pragma unroll
                                for (int kk = 0; kk < BN / 16; ++kk)      // A = P_t from tensor memory: 16 keys = 8 columns per step
                                    umma_f16_ts(tmem + TM_O + t * D, tmem + TM_P + t * (BN / 2) + 8 * kk, vd + 128 * kk, idesc_pv,
                                                (!first || kk > 0) ? 1u : 0u);
                                umma_commit(&sh->pv_done[t]);
                                jp[t]++; n_pv[t]++; progressed = true;
                            }
                        }
                    }
                    // the query tiles go back once every QK of the item is issued
                    if (!q_released && jq[0] >= w.je[0] && jq[1] >= w.je[1]) { umma_commit(&sh->q_empty[qb]); q_released = true; }
                    // a ring slot goes back once neither tile still has a QK or PV to issue on it
                    while (jr < w.j_end && !(jp[0] < w.je[0] && jp[0] <= jr) && !(jp[1] < w.je[1] && jp[1] <= jr)) {
                        umma_commit(&sh->kv_empty[(u_base + (uint32_t)(jr - w.j_begin)) % KV_STAGES]);
                        ++jr;
                    }
                    if (progressed) idle = 0;
                    else {
                        __nanosleep(32);
                        if (++idle > (SPIN_LIMIT >> 4) || ((idle & 1023u) == 0 && *abortp)) {
                            if (idle > (SPIN_LIMIT >> 4)) { *abortp = 1; atomicCAS(err, 0, 13); }
                            ok = false;
                        }
                    }
                }
                if (ok && !q_released) umma_commit(&sh->q_empty[qb]);    // an item without key tiles
                u_base += (uint32_t)(w.j_end - w.j_begin);
                for (int t = 0; t < 2; ++t) if (w.je[t] > w.jb[t]) n_act[t]++;
            }
        }
    } else if (warp >= 4) {
        // ── softmax, correction and epilogue for tile t; this thread owns one query row of the tile ──
        const int t = (warp - 4) >> 2;
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const uint32_t s_tmem = tmem + lane_base + TM_S + t * BN;
        const uint32_t p_tmem = tmem + lane_base + TM_P + t * (BN / 2);
        const uint32_t o_tmem = tmem + lane_base + TM_O + t * D;
        const float sl2 = p.scale * LOG2E;
        uint32_t n_it = 0;           // key tiles folded so far by this tile, over all items
        bool ok = true;
        int n = 0;
        for (int k = item_of_round(0); k < p.n_items && ok; k = item_of_round(++n)) {
            const Item w = make_item(p, k, nkv);
            const int r0 = w.m0 + t * BM;
            const int grow = r0 + row;                    // global query position
            float m = -INFINITY, l = 0.0f;
            for (int j = w.jb[t]; j < w.je[t] && ok; ++j, ++n_it) {
                const bool first = (j == w.jb[t]);
                ok = mbar_wait_spin(&sh->s_full[t], n_it & 1, abortp, err, 21);
                if (!ok) break;
                fence_after();
                const int k0 = j * BN;
                // does this tile straddle a mask edge for any of the 128 rows?
                bool edge = (k0 + BN > p.kv_len);
                if (p.causal || p.window > 0) edge = edge || (k0 + BN - 1 > r0);
                if (p.window > 0) edge = edge || (k0 < r0 + BM - 1 - p.window + 1);
                int klo = 0, khi = p.kv_len;              // visible keys of this row: [klo, khi)
                if (p.causal || p.window > 0) khi = min(khi, grow + 1);
                if (p.window > 0) klo = max(0, grow - p.window + 1);
                // The whole score row of this tile goes to registers in four 32-column loads; the row max of
                // one chunk is taken while the next chunk is in flight.
                uint32_t r[BN];
                float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                tmem_ld32_nowait(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    tmem_ld_wait();
                    if (c + 1 < BN / 32) tmem_ld32_nowait(s_tmem + (c + 1) * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[(c + 1) * 32]));
                    else {
                        fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh->s_free[t]);   // S_t is in registers: the next QK of this tile may overwrite it
                    }
                    if (edge) {
#pragma unroll
                        for (int i = c * 32; i < c * 32 + 32; ++i) { int kk = k0 + i; if (!(kk >= klo && kk < khi)) r[i] = 0xFF800000u; }  // -inf
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {      // four independent chains of three-input max
                        mxs[0] = max3(mxs[0], __uint_as_float(r[c * 32 + i]), __uint_as_float(r[c * 32 + i + 1]));
                        mxs[1] = max3(mxs[1], __uint_as_float(r[c * 32 + i + 2]), __uint_as_float(r[c * 32 + i + 3]));
                        mxs[2] = max3(mxs[2], __uint_as_float(r[c * 32 + i + 4]), __uint_as_float(r[c * 32 + i + 5]));
                        mxs[3] = max3(mxs[3], __uint_as_float(r[c * 32 + i + 6]), __uint_as_float(r[c * 32 + i + 7]));
                    }
                }
                const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
                // Lazy rescale: keep the reference max until the running max has moved by more than
                // 2^8; exp2(s - m_ref) then stays below 256, well inside bf16/f32 range, and o / l is
                // unchanged because both carry the same reference.
                const float m_cand = fmaxf(m, mx * sl2);
                const bool need = (m_cand - m > 8.0f) || (!(m > -INFINITY) && m_cand > -INFINITY);
                float alpha = 1.0f;
                if (need) { alpha = (m > -INFINITY) ? ex2(m - m_cand) : 0.0f; m = m_cand; }
                const float msub = (m > -INFINITY) ? m : 0.0f;
                // P = exp2(S*sl2 - m_ref) as bf16 pairs, packed in place over the score registers, and the row
                // sum. The first half is stored while the second half is still in the SFU; only at that store
                // is the previous PV of this tile needed (it has read P_t and finished O_t).
                float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
#pragma unroll
                    for (int i = hb * 32; i < hb * 32 + 32; ++i) {
                        float x0, x1;
                        ffma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), sl2, -msub);
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        fadd2(sums[(2 * i) & 7], sums[(2 * i + 1) & 7], p0, p1);
                        r[i] = pack_bf16x2(p0, p1);
                    }
                    if (hb == 0 && n_it > 0) {
                        ok = mbar_wait_spin(&sh->pv_done[t], (n_it - 1) & 1, abortp, err, 22);
                        if (!ok) break;
                        fence_after();
                        if (!first && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                            for (int c = 0; c < D / 32; ++c) {
                                uint32_t o[32];
                                tmem_ld32(o_tmem + c * 32, o);
#pragma unroll
                                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                                tmem_st32(o_tmem + c * 32, o);
                            }
                        }
                    }
                    tmem_st32(p_tmem + hb * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[hb * 32]));
                }
                if (!ok) break;
                const float sum = ((sums[0] + sums[1]) + (sums[2] + sums[3])) + ((sums[4] + sums[5]) + (sums[6] + sums[7]));
                l = l * alpha + sum;
                tmem_st_wait();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->p_full[t]);
            }
            // epilogue: read O_t back, release it for the next item, project o / l and store bf16 rows
            if (ok && w.je[t] > w.jb[t]) {
                ok = mbar_wait_spin(&sh->pv_done[t], (n_it - 1) & 1, abortp, err, 23);
                if (!ok) break;
                fence_after();
                uint32_t o[D];
                tmem_ld32_nowait(o_tmem, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
                tmem_ld32_nowait(o_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32]));
                tmem_ld_wait();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->o_free[t]);
                if (grow < p.q_len) {
                    const float inv = 1.0f / l;
                    uint16_t* dst = (uint16_t*)p.out + ((size_t)(w.b * p.q_heads + w.h) * p.q_len + grow) * D;
                    if (((uintptr_t)p.out & 31) == 0) {
                        // a 128-byte row per thread as four 32-byte stores: every lane writes whole sectors
#pragma unroll
                        for (int q = 0; q < D / 16; ++q) {
                            uint32_t wv[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                wv[j] = pack_bf16x2(__uint_as_float(o[16 * q + 2 * j]) * inv, __uint_as_float(o[16 * q + 2 * j + 1]) * inv);
                            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + q * 16), "r"(wv[0]), "r"(wv[1]),
                                         "r"(wv[2]), "r"(wv[3]), "r"(wv[4]), "r"(wv[5]), "r"(wv[6]), "r"(wv[7]) : "memory");
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < D / 8; ++q) {
                            uint32_t w0 = pack_bf16x2(__uint_as_float(o[8 * q]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
                            uint32_t w1 = pack_bf16x2(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
                            uint32_t w2 = pack_bf16x2(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
                            uint32_t w3 = pack_bf16x2(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
                            *(uint4*)(dst + q * 8) = make_uint4(w0, w1, w2, w3);
                        }
                    }
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 2) { fence_after(); tmem_dealloc(tmem, 512); }
}
}  // namespace

extern "C" int32_t sanic_attn_fwd_bf16(sanic_ctx* ctx, const sanic_attn_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->q && p->k && p->v && p->out, "attn_fwd_bf16: null tensor");
    SANIC_REQUIRE(ctx, p->batch > 0 && p->q_heads > 0 && p->kv_heads > 0 && p->q_heads % p->kv_heads == 0,
                  "attn_fwd_bf16: query heads must be a multiple of key/value heads");
    SANIC_REQUIRE(ctx, p->q_len > 0 && p->kv_len > 0, "attn_fwd_bf16: empty sequence");
    if (p->head_dim != 64 || p->v_dim != 64)
        return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "attn_fwd_bf16: head_dim and v_dim must be 64");
    SANIC_REQUIRE(ctx, !p->mask, "attn_fwd_bf16: additive masks are served by the f32 path");
    SANIC_REQUIRE(ctx, !(p->causal || p->window > 0) || p->q_len == p->kv_len,
                  "attn_fwd_bf16: causal and window masks need equal query and key lengths");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_BF16, "attn_fwd_bf16: output is bf16");
    SANIC_REQUIRE(ctx, ((uintptr_t)p->q % 16) == 0 && ((uintptr_t)p->k % 16) == 0 && ((uintptr_t)p->v % 16) == 0 &&
                  ((uintptr_t)p->out % 16) == 0, "attn_fwd_bf16: tensors must be 16-byte aligned");
    sanic_set_device(ctx);
    CUtensorMap mq, mk, mv;
    int32_t rc = sanic::tc::encode_bf16_2d(ctx, &mq, p->q, D, (uint64_t)p->batch * p->q_heads * p->q_len, D, BM);
    if (rc != SANIC_OK) return rc;
    rc = sanic::tc::encode_bf16_2d(ctx, &mk, p->k, D, (uint64_t)p->batch * p->kv_heads * p->kv_len, D, BN);
    if (rc != SANIC_OK) return rc;
    rc = sanic::tc::encode_bf16_2d(ctx, &mv, p->v, D, (uint64_t)p->batch * p->kv_heads * p->kv_len, D, BN);
    if (rc != SANIC_OK) return rc;
    const int n_mb = (p->q_len + 2 * BM - 1) / (2 * BM);
    const long long items = (long long)n_mb * p->q_heads * p->batch;
    SANIC_REQUIRE(ctx, items < (1ll << 30), "attn_fwd_bf16: too many query blocks");
    FParams fp{p->out, p->batch, p->q_heads, p->kv_heads, p->q_len, p->kv_len, p->causal, p->window, p->scale, n_mb, (int)items};
    const int smem = 4 * Q_BYTES + KV_STAGES * 2 * KV_BYTES + (int)sizeof(FShared) + 1024;
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid((unsigned)std::min<long long>(items, ctx->sm_count));   // persistent: one CTA per SM walks the item list
    attn_fwd_tc_kernel<<<grid, NTHREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, fp, ctx->status_dev);
    SANIC_LAUNCH_CHECK(ctx, "attn_fwd_bf16");
    return SANIC_OK;
}
