// Body of the split-KV decode fold, shared by the stand-alone kernel (attn_decode.cu) and the persistent
// decode-step kernel (decode_step.cu). See attn_decode.cu for the design notes.
#pragma once
#include "common.cuh"

namespace sanic {
namespace decode {

constexpr int KT = 64;        // keys per tile
constexpr int NWARP = 4;

template <int D> struct Cfg {
    static constexpr int STAGES = (D == 128) ? 3 : 4;
    static constexpr int TILE_BYTES = KT * D * 2;            // one K (or V) tile
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int MERGE_FLOATS = NWARP * 16 * (D + 2);
    static constexpr int SMEM = STAGES * STAGE_BYTES > MERGE_FLOATS * 4 ? STAGES * STAGE_BYTES : MERGE_FLOATS * 4;
};

// Issue the cp.async copies of one K tile and one V tile into a stage.
template <int D, bool VT>
__device__ __forceinline__ void load_tile(const sanic_decode_params& p, const uint16_t* Kb, const uint16_t* Vb,
                                          uint32_t stage_addr, int key0, int hi, int tid) {
    constexpr int CPR = D / 8;  // 16-byte chunks per key row
    // K tile: [D/64 halves][64 keys][128 B], chunk index xor (key & 7)
#pragma unroll
    for (int i = 0; i < (KT * CPR) / 128; ++i) {
        int id = i * 128 + tid;
        int key = id / CPR, c = id % CPR;
        int half = c >> 3, cc = c & 7;
        int gk = key0 + key;
        bool ok = gk < hi;
        const uint16_t* src = Kb + (size_t)(ok ? gk : 0) * p.k_seq_stride + c * 8;
        uint32_t dst = stage_addr + half * (KT * 128) + key * 128 + ((cc ^ (key & 7)) << 4);
        cp_async16(dst, src, ok ? 16 : 0);
    }
    uint32_t vaddr = stage_addr + Cfg<D>::TILE_BYTES;
    if (!VT) {
#pragma unroll
        for (int i = 0; i < (KT * CPR) / 128; ++i) {
            int id = i * 128 + tid;
            int key = id / CPR, c = id % CPR;
            int half = c >> 3, cc = c & 7;
            int gk = key0 + key;
            bool ok = gk < hi;
            const uint16_t* src = Vb + (size_t)(ok ? gk : 0) * p.v_row_stride + c * 8;
            uint32_t dst = vaddr + half * (KT * 128) + key * 128 + ((cc ^ (key & 7)) << 4);
            cp_async16(dst, src, ok ? 16 : 0);
        }
    } else {
        // V^T tile: [D rows][64 keys = 128 B], chunk index xor (d & 7)
#pragma unroll
        for (int i = 0; i < (D * 8) / 128; ++i) {
            int id = i * 128 + tid;
            int d = id >> 3, c = id & 7;
            int gk = key0 + c * 8;
            bool ok = gk < hi;
            const uint16_t* src = Vb + (size_t)d * p.v_row_stride + (ok ? gk : 0);
            uint32_t dst = vaddr + d * 128 + ((c ^ (d & 7)) << 4);
            // the chunk that straddles the visible edge copies only its visible keys; the rest of the 16 bytes is
            // zero-filled, so whatever the cache holds beyond the edge (NaN bit patterns included) never meets P = 0
            cp_async16(dst, src, ok ? min(16, (hi - gk) * 2) : 0);
        }
    }
}

// Barrier over the 128 threads of one item (named barrier `id`; id 0 in a 128-thread CTA is the CTA barrier).
__device__ __forceinline__ void tile_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

// Cross-device exchange folded into the fold's own last arrivers (the fused form of the multi-device step): where the
// merged raw accumulators of a (batch, kv head) group go besides carrier_out. Null pointer = single device.
struct Exchange {
    float* buf[8];               // every rank's exchange buffer as mapped here (buf[rank] is the local one)
    int rank, nranks, groups;
    unsigned epoch, spin_limit;
    void* out; int out_dtype;    // the final projected output [B, Hq, D]
};
// Layout of a fused exchange buffer, in 4-byte words: flags [2 parities][8 ranks][groups], then data
// [2 parities][nranks][rows][2 + D] (offsets are multiples of 4 words when groups is).
__host__ __device__ inline size_t xchg_flag_words(int groups) { return (size_t)2 * 8 * ((groups + 3) / 4 * 4); }

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// The visible tile range of the key axis: [T0, T1) in tiles of KT keys, keys [lo, hi).
struct KeyRange { int lo, hi, T0, T1; };
__device__ __forceinline__ KeyRange key_range(const sanic_decode_params& p, int tid, int* err) {
    // A visible length read from the device is never trusted beyond the cache extent the host vouched for: it is
    // clamped into [1, kv_cap] and the clamp is reported through the status word (the host turns code 52 into an error).
    int kv_len = p.kv_len_dev ? (*p.kv_len_dev + 1) : p.kv_len;
    if (p.kv_cap > 0 && (kv_len > p.kv_cap || kv_len < 1)) {
        kv_len = kv_len < 1 ? 1 : p.kv_cap;
        if (tid == 0 && err) atomicCAS(err, 0, 52);
    }
    KeyRange r;
    r.hi = kv_len;
    r.lo = (p.window > 0) ? max(0, kv_len - p.window) : 0;
    r.T0 = r.lo / KT;
    r.T1 = (r.hi + KT - 1) / KT;
    return r;
}

// Stage 1 of one segment: tiles [t_begin, t_end) of the key axis of (batch b, kv head hk), folded by 128 threads
// (tid in [0, 128)) into one raw accumulator per query head of the group, written to partial slot `slot` of the row.
// Then the group's ticket: returns true in the CTA that is the last of the group's `n_parts` segments to arrive (the
// partials of the whole group are then complete and visible to it). `smem_raw` is the caller's dynamic shared memory
// (Cfg<D>::SMEM bytes, 128-byte aligned); `bar_id` is the named barrier the 128 threads meet on.
template <int D, bool VT, bool SPLITP = false>
__device__ __forceinline__ bool fold_segment(const sanic_decode_params& p, int* counters, int b, int hk, int t_begin, int t_end,
                                             int lo, int hi, int slot, int n_parts, unsigned char* smem_raw, int tid, int bar_id) {
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.q_heads / p.kv_heads;
    constexpr int KS = D / 16;   // k-steps of the QK^T contraction
    constexpr int NT = D / 8;    // n-tiles of the output
    const int n_tiles = t_end - t_begin;

    const uint16_t* Kb = (const uint16_t*)p.k + (size_t)b * p.k_batch_stride + (size_t)hk * p.k_head_stride;
    const uint16_t* Vb = (const uint16_t*)p.v + (size_t)b * p.v_batch_stride + (size_t)hk * p.v_head_stride;
    const uint32_t smem_base = smem_u32(smem_raw);

    // The first tiles do not depend on q: their copies are issued before q is read, so the two latencies overlap.
    constexpr int STAGES = Cfg<D>::STAGES;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_tiles) load_tile<D, VT>(p, Kb, Vb, smem_base + s * Cfg<D>::STAGE_BYTES, (t_begin + s) * KT, hi, tid);
        cp_async_commit();
    }

    // Q fragments (read from L2: another SM may have written q earlier in the same kernel): row r = query head hk*group + r, zero beyond the group.
    uint32_t qa[KS][2];  // [ks][0] = (a0,a1) cols 2t,2t+1 ; [ks][1] = (a4,a5) cols 8+2t,+1 ; rows g (rows g+8 via qb)
    uint32_t qb[KS][2];  // rows g+8
    {
        const uint16_t* Q = (const uint16_t*)p.q + ((size_t)b * p.q_heads + (size_t)hk * group) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qa[ks][0] = (g < group) ? __ldcg((const uint32_t*)(Q + (size_t)g * D + ks * 16 + 2 * t)) : 0u;
            qa[ks][1] = (g < group) ? __ldcg((const uint32_t*)(Q + (size_t)g * D + ks * 16 + 8 + 2 * t)) : 0u;
            qb[ks][0] = (g + 8 < group) ? __ldcg((const uint32_t*)(Q + (size_t)(g + 8) * D + ks * 16 + 2 * t)) : 0u;
            qb[ks][1] = (g + 8 < group) ? __ldcg((const uint32_t*)(Q + (size_t)(g + 8) * D + ks * 16 + 8 + 2 * t)) : 0u;
        }
    }

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // rows g and g+8 (log2 units)
    const float sl2 = p.scale * LOG2E;
    for (int it = 0; it < n_tiles; ++it) {
        cp_async_wait<STAGES - 2>();
        tile_sync(bar_id);
        {   // prefetch tile it + STAGES - 1 into the stage consumed at iteration it - 1
            int nx = it + STAGES - 1;
            if (nx < n_tiles)
                load_tile<D, VT>(p, Kb, Vb, smem_base + (nx % STAGES) * Cfg<D>::STAGE_BYTES, (t_begin + nx) * KT, hi, tid);
            cp_async_commit();
        }
        const uint32_t ks_addr = smem_base + (it % STAGES) * Cfg<D>::STAGE_BYTES;
        const uint32_t vs_addr = ks_addr + Cfg<D>::TILE_BYTES;
        const int key0 = (t_begin + it) * KT + warp * 16;

        // S = Q K^T for this warp's 16 keys
        float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
        {
            const int mi = lane >> 3, r = lane & 7;
            const int krow = warp * 16 + (mi >> 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                int c = 2 * ks + (mi & 1);
                int half = c >> 3, cc = c & 7;
                uint32_t addr = ks_addr + half * (KT * 128) + krow * 128 + ((cc ^ (krow & 7)) << 4);
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4(addr, r0, r1, r2, r3);
                mma_bf16_16816(s0, qa[ks][0], qb[ks][0], qa[ks][1], qb[ks][1], r0, r1);
                mma_bf16_16816(s1, qa[ks][0], qb[ks][0], qa[ks][1], qb[ks][1], r2, r3);
            }
        }
        // mask, scale to log2 units, online-softmax update
        {
            int kA = key0 + 2 * t, kB = key0 + 8 + 2 * t;
            bool vA0 = (kA >= lo) && (kA < hi), vA1 = (kA + 1 >= lo) && (kA + 1 < hi);
            bool vB0 = (kB >= lo) && (kB < hi), vB1 = (kB + 1 >= lo) && (kB + 1 < hi);
            s0[0] = vA0 ? s0[0] * sl2 : -INFINITY; s0[1] = vA1 ? s0[1] * sl2 : -INFINITY;
            s0[2] = vA0 ? s0[2] * sl2 : -INFINITY; s0[3] = vA1 ? s0[3] * sl2 : -INFINITY;
            s1[0] = vB0 ? s1[0] * sl2 : -INFINITY; s1[1] = vB1 ? s1[1] * sl2 : -INFINITY;
            s1[2] = vB0 ? s1[2] * sl2 : -INFINITY; s1[3] = vB1 ? s1[3] * sl2 : -INFINITY;
        }
        float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
        float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a side whose max is -inf carries weight 0 (the guard of the derived combine)
        float a0 = (m0 > -INFINITY) ? exp2f(m0 - mn0) : 0.0f;
        float a1 = (m1 > -INFINITY) ? exp2f(m1 - mn1) : 0.0f;
        float sub0 = (mn0 > -INFINITY) ? mn0 : 0.0f, sub1 = (mn1 > -INFINITY) ? mn1 : 0.0f;
        float p00 = exp2f(s0[0] - sub0), p01 = exp2f(s0[1] - sub0), p10 = exp2f(s1[0] - sub0), p11 = exp2f(s1[1] - sub0);
        float p02 = exp2f(s0[2] - sub1), p03 = exp2f(s0[3] - sub1), p12 = exp2f(s1[2] - sub1), p13 = exp2f(s1[3] - sub1);
        l0 = l0 * a0 + (p00 + p01 + p10 + p11);
        l1 = l1 * a1 + (p02 + p03 + p12 + p13);
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int i = 0; i < NT; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        uint32_t pa0 = pack_bf16x2(p00, p01), pa1 = pack_bf16x2(p02, p03);
        uint32_t pa2 = pack_bf16x2(p10, p11), pa3 = pack_bf16x2(p12, p13);
        // The tensor core takes P as bf16; its rounding (2^-9 per weight) is the largest difference between this fold
        // and an f32 evaluation of the same carrier, well inside the bf16 bound. SPLITP sends the remainder
        // P - bf16(P) through a second MMA (P V = bf16(P) V + bf16(P - bf16(P)) V to 2^-17: 7e-6 instead of 1.4e-4
        // against the oracle at 2^20 keys). It is off by default: the fold is bound by HBM, but under the board's power
        // cap the extra tensor work lowers the clocks, and a sustained run measured 6.25 against 6.77 TB/s with it.
        uint32_t pl0 = 0, pl1 = 0, pl2 = 0, pl3 = 0;
        if (SPLITP) {
            pl0 = pack_bf16x2(p00 - bf16lo(pa0), p01 - bf16hi(pa0)); pl1 = pack_bf16x2(p02 - bf16lo(pa1), p03 - bf16hi(pa1));
            pl2 = pack_bf16x2(p10 - bf16lo(pa2), p11 - bf16hi(pa2)); pl3 = pack_bf16x2(p12 - bf16lo(pa3), p13 - bf16hi(pa3));
        }

        // O += P V over this warp's 16 keys
        {
            const int mi = lane >> 3, r = lane & 7;
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t addr;
                if (!VT) {
                    int krow = warp * 16 + (mi & 1) * 8 + r;
                    int c = 2 * dp + (mi >> 1);
                    int half = c >> 3, cc = c & 7;
                    addr = vs_addr + half * (KT * 128) + krow * 128 + ((cc ^ (krow & 7)) << 4);
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4_trans(addr, r0, r1, r2, r3);
                    mma_bf16_16816(o[2 * dp], pa0, pa1, pa2, pa3, r0, r1);
                    mma_bf16_16816(o[2 * dp + 1], pa0, pa1, pa2, pa3, r2, r3);
                    if (SPLITP) {
                        mma_bf16_16816(o[2 * dp], pl0, pl1, pl2, pl3, r0, r1);
                        mma_bf16_16816(o[2 * dp + 1], pl0, pl1, pl2, pl3, r2, r3);
                    }
                } else {
                    int drow = 16 * dp + (mi >> 1) * 8 + r;
                    int c = 2 * warp + (mi & 1);
                    addr = vs_addr + drow * 128 + ((c ^ (drow & 7)) << 4);
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4(addr, r0, r1, r2, r3);
                    mma_bf16_16816(o[2 * dp], pa0, pa1, pa2, pa3, r0, r1);
                    mma_bf16_16816(o[2 * dp + 1], pa0, pa1, pa2, pa3, r2, r3);
                    if (SPLITP) {
                        mma_bf16_16816(o[2 * dp], pl0, pl1, pl2, pl3, r0, r1);
                        mma_bf16_16816(o[2 * dp + 1], pl0, pl1, pl2, pl3, r2, r3);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    tile_sync(bar_id);  // every warp is done with the tile ring: reuse it for the warp merge

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    float* ms = (float*)smem_raw;  // [warp][16 rows][D + 2]
    {
        float* w0 = ms + (warp * 16 + g) * (D + 2);
        float* w1 = ms + (warp * 16 + g + 8) * (D + 2);
        if (t == 0) { w0[0] = m0; w0[1] = l0; w1[0] = m1; w1[1] = l1; }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            w0[2 + 8 * i + 2 * t] = o[i][0]; w0[2 + 8 * i + 2 * t + 1] = o[i][1];
            w1[2 + 8 * i + 2 * t] = o[i][2]; w1[2 + 8 * i + 2 * t + 1] = o[i][3];
        }
    }
    tile_sync(bar_id);
    // merge the 4 warp carriers (left to right) and write this chunk's partial
    const int W = D + 2;
    for (int idx = tid; idx < group * D; idx += 128) {
        int r = idx / D, d = idx % D;
        float m = ms[(0 * 16 + r) * W], l = ms[(0 * 16 + r) * W + 1], ov = ms[(0 * 16 + r) * W + 2 + d];
#pragma unroll
        for (int w = 1; w < NWARP; ++w) {
            float mb = ms[(w * 16 + r) * W], lb = ms[(w * 16 + r) * W + 1], ob = ms[(w * 16 + r) * W + 2 + d];
            float M = fmaxf(m, mb);
            float ra = (m > -INFINITY) ? exp2f(m - M) : 0.0f, rb = (mb > -INFINITY) ? exp2f(mb - M) : 0.0f;
            l = l * ra + lb * rb; ov = ov * ra + ob * rb; m = M;
        }
        float* part = p.partials + (((size_t)b * p.q_heads + (size_t)hk * group + r) * p.n_splits + slot) * W;
        part[2 + d] = ov;
        if (d == 0) { part[0] = m * LN2; part[1] = l; }  // m back in natural-log units
    }

    // the group's ticket: the last of its n_parts segments to arrive owns stage 2
    __shared__ int s_last;
    __threadfence();
    tile_sync(bar_id);
    if (tid == 0) {
        int ticket = atomicAdd(&counters[b * p.kv_heads + hk], 1);
        s_last = (ticket == n_parts - 1);
        if (s_last) counters[b * p.kv_heads + hk] = 0;  // ready for the next launch
    }
    tile_sync(bar_id);
    const bool last = s_last != 0;
    tile_sync(bar_id);      // s_last may be rewritten by this CTA's next segment
    if (last) __threadfence();
    return last;
}

// Stage 2 of one (batch, kv head) group, by the CTA that arrived last: merges the group's n_parts partials left to right
// with the derived combine, exports the merged raw accumulator and/or projects o / l. With an exchange, the merged raw
// accumulators are also stored into slot `rank` of every device's exchange buffer and the group's flag is published
// there (system-scope release); the cross-device merge is merge_group_remote, once the other devices' flags are in.
template <int D>
__device__ __forceinline__ void merge_group(const sanic_decode_params& p, int b, int hk, int n_parts, int tid, int bar_id,
                                            const Exchange* x) {
    const int group = p.q_heads / p.kv_heads;
    const int W = D + 2;
    const int rows = p.batch * p.q_heads;
    for (int idx = tid; idx < group * D; idx += 128) {
        int r = idx / D, d = idx % D;
        size_t row = (size_t)b * p.q_heads + (size_t)hk * group + r;
        const float* part = p.partials + row * p.n_splits * W;
        // The partials were written by other CTAs: read them from L2 (ld.global.cg), all loads
        // independent of the combine chain so their latencies overlap. The combine itself runs
        // left to right over the chunks, as stage 2 of the split reduction does.
        float m = __ldcg(part), l = __ldcg(part + 1), ov = __ldcg(part + 2 + d);
        for (int s0 = 1; s0 < n_parts; s0 += 8) {
            float mb[8], lb[8], ob[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = s0 + u < n_parts;
                const float* pb = part + (size_t)(in ? s0 + u : 0) * W;
                mb[u] = in ? __ldcg(pb) : -INFINITY; lb[u] = in ? __ldcg(pb + 1) : 0.0f; ob[u] = in ? __ldcg(pb + 2 + d) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                MloScale sc = mlo_rescale(m, mb[u]);     // an identity partial (-inf, 0, 0) is absorbed
                l = l * sc.ra + lb[u] * sc.rb; ov = ov * sc.ra + ob[u] * sc.rb; m = sc.m;
            }
        }
        if (p.carrier_out) {
            float* c = p.carrier_out + row * W;
            c[2 + d] = ov;
            if (d == 0) { c[0] = m; c[1] = l; }
        }
        if (x) {
            const size_t data_off = xchg_flag_words(x->groups) + (size_t)(x->epoch & 1) * x->nranks * rows * W;
            for (int q = 0; q < x->nranks; ++q) {
                float* c = x->buf[q] + data_off + ((size_t)x->rank * rows + row) * W;
                c[2 + d] = ov;
                if (d == 0) { c[0] = m; c[1] = l; }
            }
        } else if (p.out) {
            float v = ov / l;  // project
            if (p.out_dtype == SANIC_BF16) ((uint16_t*)p.out)[row * D + d] = f32_to_bf16_bits(v);
            else ((float*)p.out)[row * D + d] = v;
        }
    }
    if (x) {
        // every thread's peer stores are fenced before the flag that vouches for them
        __threadfence_system();
        tile_sync(bar_id);
        const int gi = b * p.kv_heads + hk;
        if (tid < x->nranks)
            st_release_sys_u32((unsigned*)x->buf[tid] + ((size_t)(x->epoch & 1) * 8 + x->rank) * ((x->groups + 3) / 4 * 4) + gi, x->epoch);
    }
}

// The cross-device half of stage 2 for one group: waits (bounded) for every device's flag of this group in the local
// exchange buffer, merges the devices' accumulators in rank order (= chunk order of the device-level split) and projects.
// Returns false when a flag never arrived (status code 41 + rank of the missing device).
template <int D>
__device__ __forceinline__ bool merge_group_remote(const sanic_decode_params& p, int b, int hk, int tid, int bar_id, const Exchange* x,
                                                   int* err) {
    const int group = p.q_heads / p.kv_heads;
    const int W = D + 2;
    const int rows = p.batch * p.q_heads;
    const int gi = b * p.kv_heads + hk;
    __shared__ int s_ok;
    if (tid == 0) {
        const unsigned* flags = (const unsigned*)x->buf[x->rank] + (size_t)(x->epoch & 1) * 8 * ((x->groups + 3) / 4 * 4);
        int ok = 1;
        for (int q = 0; q < x->nranks && ok; ++q) {
            unsigned spins = 0;
            while (ld_acquire_sys_u32(flags + (size_t)q * ((x->groups + 3) / 4 * 4) + gi) != x->epoch) {
                if (++spins > x->spin_limit) { if (err) atomicCAS(err, 0, 41 + q); ok = 0; break; }
            }
        }
        s_ok = ok;
    }
    tile_sync(bar_id);
    const bool ok = s_ok != 0;
    tile_sync(bar_id);
    if (!ok) return false;
    const float* data = x->buf[x->rank] + xchg_flag_words(x->groups) + (size_t)(x->epoch & 1) * x->nranks * rows * W;
    for (int idx = tid; idx < group * D; idx += 128) {
        int r = idx / D, d = idx % D;
        size_t row = (size_t)b * p.q_heads + (size_t)hk * group + r;
        const float* pa = data + row * W;
        float m = __ldcg(pa), l = __ldcg(pa + 1), ov = __ldcg(pa + 2 + d);
        for (int q = 1; q < x->nranks; ++q) {
            const float* pb = data + ((size_t)q * rows + row) * W;
            const MloScale sc = mlo_rescale(m, __ldcg(pb));
            l = l * sc.ra + __ldcg(pb + 1) * sc.rb; ov = ov * sc.ra + __ldcg(pb + 2 + d) * sc.rb; m = sc.m;
        }
        const float v = ov / l;
        if (x->out_dtype == SANIC_BF16) ((uint16_t*)x->out)[row * D + d] = f32_to_bf16_bits(v);
        else ((float*)x->out)[row * D + d] = v;
    }
    return true;
}

// One (chunk, kv head, batch) item of the fold in its fixed-chunk form: chunk `split` of n_splits equal tile ranges,
// executed by 128 threads (tid in [0, 128)); `pdl` as in gemv_tile.
template <int D, bool VT, bool SPLITP = false>
__device__ __forceinline__ void attn_decode_tile(const sanic_decode_params& p, int* counters, int split, int hk, int b,
                                                 unsigned char* smem_raw, int tid, bool pdl, int bar_id, int* err) {
    if (pdl) { griddep_launch(); griddep_wait(); }   // q, the caches and the position come from the previous kernels of the step
    const KeyRange kr = key_range(p, tid, err);
    const int nT = kr.T1 - kr.T0;
    const int t_begin = kr.T0 + (int)(((long long)split * nT) / p.n_splits);
    const int t_end = kr.T0 + (int)(((long long)(split + 1) * nT) / p.n_splits);
    if (fold_segment<D, VT, SPLITP>(p, counters, b, hk, t_begin, t_end, kr.lo, kr.hi, split, p.n_splits, smem_raw, tid, bar_id))
        merge_group<D>(p, b, hk, p.n_splits, tid, bar_id, nullptr);
}

// Host side: the argument checks of one split-KV fold.
inline int32_t host_validate(sanic_ctx* ctx, const sanic_decode_params* p) {
    SANIC_REQUIRE(ctx, p->q && p->k && p->v && p->partials, "attn_decode: null tensor or scratch");
    SANIC_REQUIRE(ctx, p->out || p->carrier_out, "attn_decode: no output requested");
    SANIC_REQUIRE(ctx, p->head_dim == 64 || p->head_dim == 128, "attn_decode: head_dim must be 64 or 128");
    SANIC_REQUIRE(ctx, p->batch > 0 && p->kv_heads > 0 && p->q_heads % p->kv_heads == 0 &&
                  p->q_heads / p->kv_heads <= 16, "attn_decode: GQA group must divide and be <= 16");
    SANIC_REQUIRE(ctx, p->n_splits >= 1, "attn_decode: n_splits must be >= 1");
    SANIC_REQUIRE(ctx, p->kv_len_dev || p->kv_len >= 1, "attn_decode: empty key axis");
    SANIC_REQUIRE(ctx, p->kv_cap >= 0 && (!p->kv_len_dev || p->kv_cap >= 1),
                  "attn_decode: a device-side length needs kv_cap, the key extent of the cache");
    SANIC_REQUIRE(ctx, p->kv_cap == 0 || p->kv_len_dev || p->kv_len <= p->kv_cap, "attn_decode: kv_len exceeds kv_cap");
    if (p->kv_cap > 0) {
        // kv_cap keys must fit inside one (batch, kv head) slice as the strides describe it
        const int64_t k_span = (int64_t)p->kv_cap * p->k_seq_stride;
        const bool k_head_major = p->k_head_stride >= p->k_seq_stride;      // [.., head, seq, D]; else [.., seq, head, D]
        SANIC_REQUIRE(ctx, !k_head_major || ((p->kv_heads == 1 || k_span <= p->k_head_stride) && (p->batch == 1 || k_span <= p->k_batch_stride)),
                      "attn_decode: kv_cap keys do not fit the K strides");
        if (p->v_transposed) {
            SANIC_REQUIRE(ctx, p->kv_cap <= p->v_row_stride, "attn_decode: kv_cap keys do not fit a row of the transposed V");
        } else {
            const int64_t v_span = (int64_t)p->kv_cap * p->v_row_stride;
            const bool v_head_major = p->v_head_stride >= p->v_row_stride;
            SANIC_REQUIRE(ctx, !v_head_major || ((p->kv_heads == 1 || v_span <= p->v_head_stride) && (p->batch == 1 || v_span <= p->v_batch_stride)),
                          "attn_decode: kv_cap keys do not fit the V strides");
        }
    }
    SANIC_REQUIRE(ctx, p->k_seq_stride % 8 == 0 && p->k_head_stride % 8 == 0 && p->k_batch_stride % 8 == 0 &&
                  p->v_row_stride % 8 == 0 && p->v_head_stride % 8 == 0 && p->v_batch_stride % 8 == 0 &&
                  ((uintptr_t)p->k % 16) == 0 && ((uintptr_t)p->v % 16) == 0 && ((uintptr_t)p->q % 4) == 0,
                  "attn_decode: K/V rows must be 16-byte aligned");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_F32 || p->out_dtype == SANIC_BF16 || !p->out, "attn_decode: bad out dtype");
    return SANIC_OK;
}

}  // namespace decode
}  // namespace sanic
