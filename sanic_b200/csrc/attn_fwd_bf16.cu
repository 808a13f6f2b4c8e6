// Online-softmax fold for prefill (FlashAttention forward), bf16 storage, head_dim 64, on the
// 5th-generation tensor cores: S = Q K^T and O += P V are tcgen05 MMAs with TMEM accumulators,
// Q/K/V tiles arrive by TMA, and the (m, l, o) carrier of each query row is kept by the thread that
// owns that row (one TMEM lane per row, so row max and row sum need no shuffles).
//
// One CTA folds 256 query rows of one (batch, query head) as two 128-row tiles that ping-pong on
// the tensor core: while one tile's softmax warpgroup turns S into P, the other tile's MMAs run.
//   warp 0       TMA producer: Q once, then K_j / V_j tiles of 128 keys through a 5-stage ring
//   warps 1, 3   MMA issuers, one warp per query tile (an elected lane issues): QK(t,j+1) when S(t,j) is in registers,
//                PV(t,j) when P(t,j) is stored
//   warp 2       TMEM allocator (S0 S1 | P0 P1 | O0 O1 = 2x128 + 2x64 + 2x64 columns, all 512)
//   warps 4-7    softmax + correction + epilogue of tile 0
//   warps 8-11   the same for tile 1
// P never touches shared memory: the softmax threads write bf16 pairs back to tensor memory and
// the PV MMA takes its A operand from there.
// Masks: causal (key > row), sliding window (key < row - window + 1) and the ragged key tail are
// applied only in tiles that straddle an edge; tiles wholly outside the visible range are never
// loaded (a prefix-masked fold may stop at the mask edge: it contributes exact zeros).
// The rescale of O by exp(m_old - m_new) is skipped when no row of the warp moved its max, and after an item's first
// key tile the row maximum is taken inside the first half of the exponentials (redone if a reference did move).
// The first warpgroup hands registers to the softmax warpgroups (setmaxnreg: 56 / 224 per thread).
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

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ uint32_t clock32() {
    uint32_t c;
    asm volatile("mov.u32 %0, %%clock;" : "=r"(c)::"memory");
    return c;
}

// PROF: the softmax warp of rows 0-31 of each tile, and the MMA thread, of CTA 0 count clocks per part of their loops
// (prof[0..11] tile 0, [12..23] tile 1, [24..31] and [32..39] the MMA threads); the results are computed and stored all the same.
template <bool PROF>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, FParams p, int* err, unsigned long long* prof) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* aligned = smem_dyn + (base - raw);
    const uint32_t q_addr = base, kv_addr = base + 4 * Q_BYTES;
    FShared* sh = (FShared*)(aligned + 4 * Q_BYTES + KV_STAGES * 2 * KV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkv = (p.kv_len + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) { mbar_init(&sh->q_full[i], 1); mbar_init(&sh->q_empty[i], 2); }
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&sh->k_full[s], 1); mbar_init(&sh->v_full[s], 1); mbar_init(&sh->kv_empty[s], 2); }
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
    // The softmax threads hold a whole 128-score row each: the first warpgroup (producer, MMA issuers, allocator) gives
    // registers up and the two softmax warpgroups take them (128 x 56 + 256 x 224 = the 64,512 the launch was given).

    // Every role walks the same item sequence: its own sub-list; all barrier
    // parities come from running counts, so nothing is re-initialised between items.
    if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
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
    } else if (warp == 1 || warp == 3) {
        {
            // The whole warp walks the role with warp-uniform control flow (barrier answers are made uniform by a vote) and
            // one elected lane issues: the descriptors can then live in uniform registers (an MMA took 90 clocks to issue
            // from a single diverged thread, 40 this way).
            const bool leader = elect_one();
            // One MMA-issuing warp per query tile (warp 1: tile 0, warp 3: tile 1), each serving its tile's two events
            // (S free -> next QK, P full -> PV) in arrival order: a single thread serving both tiles spent its whole time
            // in barrier tests and MMA issue (1950 clocks per key tile of each query tile). QK(t, j+1) is issued as soon as tile
            // t's softmax warps have pulled S(t, j) into registers, so the next scores are ready before the exponentials
            // of the current ones finish; PV(t, j) follows when P(t, j) is written. A ring slot and the query tiles go back
            // to the producer when both threads have handed them back (barrier counts of 2).
            const int t = __shfl_sync(0xffffffffu, warp == 3 ? 1 : 0, 0);
            constexpr uint32_t idesc_qk = make_idesc(BM, BN, false);
            constexpr uint32_t idesc_pv = make_idesc(BM, D, true);
            bool ok = true;
            int n = 0;
            uint32_t u_base = 0;                 // key tiles of all earlier items: position in the K/V ring
            uint32_t n_qk = 0, n_pv = 0;         // QK / PV issues so far, over all items
            uint32_t n_act = 0;                  // earlier items in which the tile had work (its O was read back)
            uint32_t polls = 0, idle_polls = 0, mc[4] = {0, 0, 0, 0};
            const uint32_t mma_t0 = PROF ? clock32() : 0u;
            uint32_t m_mark = mma_t0;
#define SANIC_MTICK(i) do { if (PROF) { const uint32_t now_ = clock32(); mc[i] += now_ - m_mark; m_mark = now_; } } while (0)
            for (int k = item_of_round(0); k < p.n_items && ok; k = item_of_round(++n)) {
                const Item w = make_item(p, k, nkv);
                const int qb = n & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&sh->q_full[qb], (n >> 1) & 1, abortp, err, 12));
                if (!ok) break;
                fence_after();
                const bool active = w.je[t] > w.jb[t];
                const int lo = active ? max(w.jb[t], w.j_begin) : w.j_begin;
                const int hi = active ? min(w.je[t], w.j_end) : w.j_begin;
                // A key tile of the item that this query tile does not see goes back untouched. The arrival may only count
                // for the slot's current use: its previous use must have been handed back by both threads first.
                auto hand_back_unused = [&](int j) -> bool {
                    const uint32_t u = u_base + (uint32_t)(j - w.j_begin);
                    const int stage = u % KV_STAGES;
                    if (u >= (uint32_t)KV_STAGES && !__all_sync(0xffffffffu, mbar_wait(&sh->kv_empty[stage], ((u / KV_STAGES) - 1) & 1, abortp, err, 14))) return false;
                    if (leader) mbar_arrive(&sh->kv_empty[stage]);
                    return true;
                };
                for (int j = w.j_begin; j < lo && ok; ++j) ok = hand_back_unused(j);
                if (!active && ok && leader) mbar_arrive(&sh->q_empty[qb]);      // no rows of this tile in the item
                int jq = lo;      // next key tile whose QK is to be issued
                int jp = lo;      // next key tile whose PV is to be issued
                uint32_t idle = 0;
                SANIC_MTICK(3);
                while (ok && jp < hi) {
                    bool progressed = false;
                    if (jq < hi) {
                        const uint32_t u = u_base + (uint32_t)(jq - w.j_begin);
                        const int stage = u % KV_STAGES;
                        if (__all_sync(0xffffffffu, (n_qk == 0 || mbar_test(&sh->s_free[t], (n_qk - 1) & 1)) && mbar_test(&sh->k_full[stage], (u / KV_STAGES) & 1))) {
                            fence_after();
                            SANIC_MTICK(0);
                            const uint64_t ad = make_desc(q_addr + (qb * 2 + t) * Q_BYTES, 16, 1024);
                            const uint64_t bd = make_desc(kv_addr + stage * 2 * KV_BYTES, 16, 1024);
#pragma unroll
                            for (int kk = 0; kk < D / 16; ++kk) if (leader) umma_f16(tmem + TM_S + t * BN, ad + 2 * kk, bd + 2 * kk, idesc_qk, kk > 0 ? 1u : 0u);
                            if (leader) umma_commit(&sh->s_full[t]);
                            jq++; n_qk++; progressed = true;
                            if (jq == hi && leader) umma_commit(&sh->q_empty[qb]);     // every QK of the item is issued: the query tile goes back
                            SANIC_MTICK(1);
                        }
                    }
                    if (jp < jq) {
                        const uint32_t u = u_base + (uint32_t)(jp - w.j_begin);
                        const int stage = u % KV_STAGES;
                        const bool first = (jp == lo);
                        // the first PV of an item overwrites O_t: the epilogue of the tile's previous item must have read it
                        if (__all_sync(0xffffffffu, mbar_test(&sh->p_full[t], n_pv & 1) && mbar_test(&sh->v_full[stage], (u / KV_STAGES) & 1) &&
                                                     (!first || n_act == 0 || mbar_test(&sh->o_free[t], (n_act - 1) & 1)))) {
                            fence_after();
                            SANIC_MTICK(0);
                            const uint64_t vd = make_desc(kv_addr + stage * 2 * KV_BYTES + KV_BYTES, 1024, 1024);
#pragma unroll
                            for (int kk = 0; kk < BN / 16; ++kk)      // A = P_t from tensor memory: 16 keys = 8 columns per step
                                if (leader) umma_f16_ts(tmem + TM_O + t * D, tmem + TM_P + t * (BN / 2) + 8 * kk, vd + 128 * kk, idesc_pv,
                                            (!first || kk > 0) ? 1u : 0u);
                            if (leader) umma_commit(&sh->pv_done[t]);
                            if (leader) umma_commit(&sh->kv_empty[stage]);      // this tile's QK and PV on the slot are issued
                            jp++; n_pv++; progressed = true;
                            SANIC_MTICK(2);
                        }
                    }
                    SANIC_MTICK(0);
                    if (PROF) { ++polls; if (!progressed) ++idle_polls; }
                    if (progressed) idle = 0;
                    else {
                        __nanosleep(32);
                        if (++idle > (SPIN_LIMIT >> 4) || ((idle & 1023u) == 0 && __any_sync(0xffffffffu, *abortp != 0))) {
                            if (idle > (SPIN_LIMIT >> 4) && leader) { *abortp = 1; atomicCAS(err, 0, 13); }
                            ok = false;
                        }
                    }
                }
                for (int j = hi; j < w.j_end && ok; ++j) ok = hand_back_unused(j);
                SANIC_MTICK(3);
                u_base += (uint32_t)(w.j_end - w.j_begin);
                if (active) n_act++;
            }
            if (PROF && blockIdx.x == 0 && leader) {
                unsigned long long* o = prof + 24 + 8 * t;
                o[0] = polls; o[1] = idle_polls; o[2] = clock32() - mma_t0; o[3] = n_qk;
                for (int i = 0; i < 4; ++i) o[4 + i] = mc[i];
            }
#undef SANIC_MTICK
        }
    } else if (warp >= 4) {
        // ── softmax, correction and epilogue for tile t; this thread owns one query row of the tile ──
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
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
        // Each of the loop's two waits is asked ahead of time, with exponentials between the question and the use of its
        // answer; the bounded wait (a loop with its abort checks) runs only when the early answer was no.
        bool scores_ready = false;
        uint32_t pc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0}, t_mark = PROF ? clock32() : 0u;
        const uint32_t t_start = t_mark;
#define SANIC_TICK(i) do { if (PROF) { const uint32_t now_ = clock32(); pc[i] += now_ - t_mark; t_mark = now_; } } while (0)
        for (int k = item_of_round(0); k < p.n_items && ok; k = item_of_round(++n)) {
            const Item w = make_item(p, k, nkv);
            const int r0 = w.m0 + t * BM;
            const int grow = r0 + row;                    // global query position
            float m = -INFINITY, l = 0.0f;
            for (int j = w.jb[t]; j < w.je[t] && ok; ++j, ++n_it) {
                const bool first = (j == w.jb[t]);
                SANIC_TICK(8);
                if (!scores_ready) {
                    ok = mbar_wait_spin(&sh->s_full[t], n_it & 1, abortp, err, 21);
                    if (!ok) break;
                }
                SANIC_TICK(0);
                fence_after();
                SANIC_TICK(9);
                const int k0 = j * BN;
                // does this tile straddle a mask edge for any of the 128 rows?
                bool edge = (k0 + BN > p.kv_len);
                if (p.causal || p.window > 0) edge = edge || (k0 + BN - 1 > r0);
                if (p.window > 0) edge = edge || (k0 < r0 + BM - 1 - p.window + 1);
                int klo = 0, khi = p.kv_len;              // visible keys of this row: [klo, khi)
                if (p.causal || p.window > 0) khi = min(khi, grow + 1);
                if (p.window > 0) klo = max(0, grow - p.window + 1);
                // The whole score row of this tile goes to registers: four 32-column loads in flight together, one wait.
                uint32_t r[BN];
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) tmem_ld32_nowait(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
                tmem_ld_wait();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->s_free[t]);   // S_t is in registers: the next QK of this tile may overwrite it
                SANIC_TICK(1);
                if (edge) {
#pragma unroll
                    for (int i = 0; i < BN; ++i) { int kk = k0 + i; if (!(kk >= klo && kk < khi)) r[i] = 0xFF800000u; }  // -inf
                }
                // Lazy rescale: the reference max is kept until the running max has moved by more than 2^8; exp2(s - m_ref)
                // then stays below 256, well inside bf16/f32 range, and o / l is unchanged because both carry the same
                // reference. So after an item's first key tile the reference almost never moves, and the row maximum (64
                // three-input max instructions, about 500 clocks on their own) is taken inside the first half of the
                // exponentials, where the SFU sets the pace: that half runs against the old reference, and is redone (its
                // scores stay in registers: the half's bf16 pairs go to registers of their own) in the rare case that some
                // row's reference did move.
                // The first key tile has no reference yet: its maximum comes first. Under a sliding window so does the second's:
                // the rows whose window opens after the first key tile still have none.
                const bool spec = !first && !(p.window > 0 && j == w.jb[t] + 1);
                float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                float alpha = 1.0f;
                bool need = false;
                auto new_reference = [&]() {
                    const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
                    const float m_cand = fmaxf(m, mx * sl2);
                    need = (m_cand - m > 8.0f) || (!(m > -INFINITY) && m_cand > -INFINITY);
                    if (need) { alpha = (m > -INFINITY) ? ex2(m - m_cand) : 0.0f; m = m_cand; }
                };
                if (!spec) {
#pragma unroll
                    for (int i = 0; i < BN; i += 8) {      // four independent chains of three-input max
                        mxs[0] = max3(mxs[0], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                        mxs[1] = max3(mxs[1], __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                        mxs[2] = max3(mxs[2], __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                        mxs[3] = max3(mxs[3], __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                    }
                    new_reference();
                }
                SANIC_TICK(2);
                float msub = (m > -INFINITY) ? m : 0.0f;
                const bool pv_ready = n_it > 0 && mbar_test(&sh->pv_done[t], (n_it - 1) & 1);
                // P = exp2(S*sl2 - m_ref) as bf16 pairs, packed in place over the score registers, and the row
                // sum. The first half is stored while the second half is still in the SFU; only at that store
                // is the previous PV of this tile needed (it has read P_t and finished O_t).
                float sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                uint32_t pk[32];        // the first half's pairs
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (spec) {     // the row maximum of all 128 scores, four per step
                        mxs[0] = max3(mxs[0], __uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]));
                        mxs[1] = max3(mxs[1], __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                    }
                    float x0, x1;
                    ffma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), sl2, -msub);
                    const float p0 = ex2(x0), p1 = ex2(x1);
                    fadd2(sums[(2 * i) & 7], sums[(2 * i + 1) & 7], p0, p1);
                    pk[i] = pack_bf16x2(p0, p1);
                }
                if (spec) {
                    new_reference();
                    if (__any_sync(0xffffffffu, need)) {
                        // some row's reference moved: the half is taken again against the new one
                        msub = (m > -INFINITY) ? m : 0.0f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) sums[i] = 0.0f;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float x0, x1;
                            ffma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), sl2, -msub);
                            const float p0 = ex2(x0), p1 = ex2(x1);
                            fadd2(sums[(2 * i) & 7], sums[(2 * i + 1) & 7], p0, p1);
                            pk[i] = pack_bf16x2(p0, p1);
                        }
                    }
                }
                if (n_it > 0) {
                    SANIC_TICK(3);
                    if (!pv_ready) {
                        ok = mbar_wait_spin(&sh->pv_done[t], (n_it - 1) & 1, abortp, err, 22);
                        if (!ok) break;
                    }
                    fence_after();
                    SANIC_TICK(4);
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
                    SANIC_TICK(5);
                }
                tmem_st32(p_tmem, pk);
                scores_ready = (j + 1 < w.je[t]) && mbar_test(&sh->s_full[t], (n_it + 1) & 1);     // the next key tile's scores
#pragma unroll
                for (int i = 32; i < 64; ++i) {
                    float x0, x1;
                    ffma2(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), sl2, -msub);
                    const float p0 = ex2(x0), p1 = ex2(x1);
                    fadd2(sums[(2 * i) & 7], sums[(2 * i + 1) & 7], p0, p1);
                    r[i] = pack_bf16x2(p0, p1);
                }
                tmem_st32(p_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                if (!ok) break;
                const float sum = ((sums[0] + sums[1]) + (sums[2] + sums[3])) + ((sums[4] + sums[5]) + (sums[6] + sums[7]));
                l = l * alpha + sum;
                SANIC_TICK(6);
                tmem_st_wait();
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->p_full[t]);
                SANIC_TICK(7);
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
        if (PROF && blockIdx.x == 0 && q4 == 0 && lane == 0) {
            SANIC_TICK(8);
            for (int i = 0; i < 10; ++i) prof[t * 12 + i] = pc[i];
            prof[t * 12 + 10] = n_it;
            prof[t * 12 + 11] = t_mark - t_start;
        }
#undef SANIC_TICK
    }
    fence_before();
    __syncthreads();
    if (warp == 2) { fence_after(); tmem_dealloc(tmem, 512); }
}
}  // namespace

static int32_t attn_fwd_launch(sanic_ctx* ctx, const sanic_attn_params* p, void* stream, unsigned long long* prof) {
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
    dim3 grid((unsigned)std::min<long long>(items, ctx->sm_count));   // persistent: one CTA per SM walks the item list
    if (prof) {
        SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attn_fwd_tc_kernel<true><<<grid, NTHREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, fp, ctx->status_dev, prof);
    } else {
        SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(attn_fwd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attn_fwd_tc_kernel<false><<<grid, NTHREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, fp, ctx->status_dev, nullptr);
    }
    SANIC_LAUNCH_CHECK(ctx, "attn_fwd_bf16");
    return SANIC_OK;
}

extern "C" int32_t sanic_attn_fwd_bf16(sanic_ctx* ctx, const sanic_attn_params* p, void* stream) {
    return attn_fwd_launch(ctx, p, stream, nullptr);
}

extern "C" int32_t sanic_attn_fwd_bf16_profile(sanic_ctx* ctx, const sanic_attn_params* p, void* stream, uint64_t* out) {
    if (!ctx || !p || !out) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    unsigned long long* d = nullptr;
    SANIC_CUDA_CHECK(ctx, cudaMalloc(&d, 40 * sizeof(unsigned long long)));
    cudaError_t e = cudaMemsetAsync(d, 0, 40 * sizeof(unsigned long long), (cudaStream_t)stream);
    int32_t rc = e == cudaSuccess ? attn_fwd_launch(ctx, p, stream, d) : SANIC_ERR_CUDA;
    if (rc == SANIC_OK) {
        e = cudaMemcpyAsync(out, d, 40 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
        if (e != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, cudaGetErrorString(e));
    }
    cudaFree(d);
    return rc;
}
