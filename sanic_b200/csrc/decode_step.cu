// One decode step as one persistent, cooperatively launched, warp-specialised kernel.
//
// A captured launch list pays a fixed cost per kernel (launch, ramp-up, drain) that is several times
// the HBM time of a decode-step stage: a 2048x2048 bf16 projection is 8 MB, 1.3 us of bandwidth. Here
// the stage list (reference src/partition.rs:101-127) is lowered once into a table of phases; one block
// per SM walks the table, each phase strided over the blocks, with a grid-wide barrier where the launch
// list had a kernel boundary.
//
//   warps 0-7   consumers: run the phase bodies. A contraction takes its weight fragments from a
//               shared-memory ring and its activations from a per-phase shared-memory copy (RMSNorm applied
//               while staging), then sums the warps and runs the epilogue exactly as the stand-alone kernel
//               does (gemv_body.cuh: tile_finish). Attention phases run the stand-alone fold body
//               (attn_decode_body.cuh) on a named barrier.
//   warps 8-11  producers: stream the weights of EVERY contraction phase, in consumption order, into the ring
//               with cp.async.bulk row copies that complete on mbarriers (ring slots dealt round-robin to the
//               four warps: one warp cannot issue copies fast enough). Weights are constant within a step, so
//               the producers run ahead of the grid barriers: HBM keeps streaming while the consumers wait for
//               activations, which a launch list cannot do.
//
// Both forms of a step compute the same values (same fragment layout, same summation order per tile). Data
// written in one phase and read in a later one crosses SMs inside one kernel: those reads go to L2
// (ld.global.cg), never through the non-coherent L1.
//
// The grid barrier is a monotonic arrival counter (cleared on the stream before the launch): release-add,
// acquire-poll. Every spin (grid barrier, ring mbarriers) is bounded: a block that gives up raises the abort
// word, records a code in the context's status word and leaves; the others see the abort word or run out of
// spins themselves, and no block exits while a bulk copy into its shared memory is still in flight.
//
// The same producer and consumer halves also run as a kernel of their own, one contraction per launch
// (gemv_ring_kernel, used by launch lists at batch 9-16): one producer warp, activations read through L1 instead of
// staged, and for bf16 blocks small enough that two share an SM, so that the next kernel's producers stream weights
// while this kernel drains.
#include "decode_step.cuh"

#include <algorithm>
#include <new>

#include "attn_decode_body.cuh"
#include "gemv_body.cuh"

namespace sanic {
namespace step {
namespace {

enum { PH_GEMV = 1, PH_DECODE, PH_EMBED, PH_RMSNORM, PH_ARGMAX_PART, PH_ARGMAX_FINAL, PH_ADVANCE };
constexpr int CONSUMERS = 256;              // warps 0-7: the phase bodies
constexpr int PRODUCERS = 4;                // warps 8..: the weight producers, ring stages dealt round-robin
constexpr int THREADS = CONSUMERS + 32 * PRODUCERS;
constexpr int RING_THREADS = CONSUMERS + 32;   // the stand-alone ring-fed contraction: one producer warp
constexpr int AMAX_CHUNKS = 128;
constexpr unsigned SPIN_LIMIT = 1u << 22;
constexpr int SLOTS = 4;                    // weight ring
constexpr int SLOT_BYTES = 35840;           // the largest stage: 32 int4 rows x (1024 + 32) B + 32 x 64 B of scales
constexpr int SCRATCH_BYTES = 20480;        // contraction scratch (row norms, cross-warp sums) | pointwise scratch
constexpr int XS_BYTES = 66560;             // a phase's activations, bf16, norm applied: 16 rows x (2048 + 32) x 2 B
constexpr int SHARED_BYTES = SCRATCH_BYTES + XS_BYTES;   // the attention K/V ring overlays both
constexpr int RING_BYTES = SLOTS * SLOT_BYTES;

struct Phase {
    int op, n_blocks;
    int variant;                 // GEMV: bit0 int4, bit1 batch > 8, bit2 silu-mul pair, bit3 inlined norm; DECODE: bit0 V transposed
    // contraction
    const uint16_t* x; int batch, K;
    gemv::SegTable segs; int n_segments, out_dtype, epilogue; const float* residual; gemv::Fused fz;
    // split-KV fold
    sanic_decode_params dec; int* counters;
    // pointwise / gather / extremum index
    const void* a; const void* b; void* c; float* scratch;
    int i0, i1, i2; float f0;
};

// One ring stage of a contraction: `rows` weight rows (16, or 32 for the silu-mul pair) x `stage_k` inputs, about
// 32 KB, each row one bulk copy of 1-2 KB; int4 stages carry their bf16 group scales behind the weights.
struct Geom { int stage_k, n_stages, rows, row_bytes, pitch, scale_off, scale_row_bytes; };
__host__ __device__ inline Geom geom_of(bool w4, bool dual, int K) {
    Geom g;
    const int cap = (dual ? 512 : 1024) * (w4 ? 4 : 1);
    g.stage_k = K < cap ? K : cap;
    g.n_stages = K / g.stage_k;
    g.rows = dual ? 32 : 16;
    g.row_bytes = w4 ? g.stage_k / 2 : g.stage_k * 2;
    // rows land 4 bank groups apart: conflict-free fragment reads. An int4 stage that holds whole rows is dense instead: the 16
    // rows of a tile are then one contiguous piece of the matrix and arrive as ONE bulk copy (a 1 KB copy per row and a
    // 64-byte one per scale row kept the copy engine, not HBM, busy); the fragment reads pay bank conflicts for it.
    g.pitch = g.row_bytes + (w4 ? (g.n_stages == 1 ? 0 : 32) : 64);
    g.scale_off = g.rows * g.pitch;
    g.scale_row_bytes = (w4 && g.stage_k >= 512) ? g.stage_k / 64 * 2 : 0;   // 0: too short for a bulk copy, read from global
    return g;
}

// k values per staged activation row when a phase's activations do not fit the staging area whole: a ring stage,
// halved until `batch` rows of it (plus the row padding) fit
__host__ __device__ inline int stage_span(int batch, int stage_k) {
    int span = stage_k;
    while (span > 64 && (size_t)batch * (span * 2 + 64) > (size_t)XS_BYTES) span >>= 1;
    return span;
}

// weight row (within its matrix) of fragment row r (0..15) of row tile `tile`
__device__ __forceinline__ int weight_row(int epilogue, const gemv::Fused& fz, int tile, int r) {
    if (epilogue == SANIC_EPI_ROPE_CACHE) {      // rotate-half partners d = 8*sub + r and d + D/2 of one head
        const int tph = fz.head_dim / 16, head = tile / tph, sub = tile % tph;
        return head * fz.head_dim + 8 * sub + (r & 7) + (r >= 8 ? fz.head_dim / 2 : 0);
    }
    return tile * 16 + r;
}
__device__ __forceinline__ void seg_of_tile(const gemv::SegTable& segs, int n_segments, bool dual, int gtile, int& seg, int& tile) {
    seg = 0;
    if (!dual) {
        if (n_segments > 1 && gtile >= segs.tile_begin[1]) seg = 1;
        if (n_segments > 2 && gtile >= segs.tile_begin[2]) seg = 2;
    }
    tile = gtile - (seg == 0 ? segs.tile_begin[0] : (seg == 1 ? segs.tile_begin[1] : segs.tile_begin[2]));
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// bar[0]: arrivals so far in this launch, bar[1]: abort word. Every wait below is bounded and gives up when the
// abort word is set; the one that runs out of spins sets it and records a code in the status word.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned* gbar, int* err, int code) {
    for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_test(bar, parity)) return true;
        if (gbar && (it & 4095u) == 4095u && ld_acquire(gbar + 1) != 0) return false;
    }
    if (gbar) atomicExch(gbar + 1, 1u);
    atomicCAS(err, 0, code);
    return false;
}
// one contiguous row piece, global -> shared, completion counted in bytes on an mbarrier of this CTA
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }

// Block 0 leaves a clock stamp (profile of the phase it is in; null = off)
__device__ __forceinline__ void stamp(unsigned long long* prof, int slot) {
    if (prof && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long g;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
        prof[slot] = g;
    }
}

__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned target, int* err, int* s_ok) {
    consumer_sync();
    if (threadIdx.x == 0) {
        // Release-arrive without waiting for the old value, then acquire-poll: the block barrier before orders the
        // other threads' writes ahead of this release, the one after hands the acquired view to them.
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
        int ok = 1;
        unsigned spins = 0;
        while (ld_acquire(bar) < target) {
            if ((++spins & 63u) == 0 && ld_acquire(bar + 1) != 0) { ok = 0; break; }
            if (spins > SPIN_LIMIT) { atomicExch(bar + 1, 1u); atomicCAS(err, 0, 31); ok = 0; break; }
        }
        *s_ok = ok;
    }
    consumer_sync();
    return *s_ok != 0;
}

struct Ring {
    uint64_t* full; uint64_t* empty;     // [SLOTS] each
    uint32_t base;                       // shared-memory address of slot 0
    unsigned char* ptr;                  // generic pointer to slot 0
};

// RMSNorm of up to two rows of 2048 values, staged as bf16 in shared memory, in one pass: thread t holds 8 consecutive
// values of every row, so the sum of squares and the normalised row come from the same loads (one L2 round trip, not
// two). Kept out of line: its live registers must not add to the contraction loop's.
__device__ __noinline__ void stage_normed_rows(const Phase& P, float* scratch, unsigned char* xs, int xpitch) {
    using namespace gemv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
        float (*s_part)[GW] = reinterpret_cast<float (*)[GW]>(scratch + 16);
        float4 xa[2], xb[2];
        const uint4 gm = __ldg((const uint4*)(P.fz.norm_gamma + tid * 8));
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            if (n >= P.batch) break;
            xa[n] = __ldcg((const float4*)(P.fz.norm_x + (size_t)n * P.K + tid * 8));
            xb[n] = __ldcg((const float4*)(P.fz.norm_x + (size_t)n * P.K + tid * 8 + 4));
        }
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            if (n >= P.batch) break;
            float ss = xa[n].x * xa[n].x;
            ss = fmaf(xa[n].y, xa[n].y, ss); ss = fmaf(xa[n].z, xa[n].z, ss); ss = fmaf(xa[n].w, xa[n].w, ss);
            ss = fmaf(xb[n].x, xb[n].x, ss); ss = fmaf(xb[n].y, xb[n].y, ss); ss = fmaf(xb[n].z, xb[n].z, ss); ss = fmaf(xb[n].w, xb[n].w, ss);
            ss = warp_sum(ss);
            if (lane == 0) s_part[n][warp] = ss;
        }
        consumer_sync();
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            if (n >= P.batch) break;
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < GW; ++w) tot += s_part[n][w];
            const float den = 1.0f / sqrtf(tot * (1.0f / (float)P.K) + P.fz.norm_eps);
            uint4 r;
            r.x = pack_bf16x2((xa[n].x * bf16lo(gm.x)) * den, (xa[n].y * bf16hi(gm.x)) * den);
            r.y = pack_bf16x2((xa[n].z * bf16lo(gm.y)) * den, (xa[n].w * bf16hi(gm.y)) * den);
            r.z = pack_bf16x2((xb[n].x * bf16lo(gm.z)) * den, (xb[n].y * bf16hi(gm.z)) * den);
            r.w = pack_bf16x2((xb[n].z * bf16lo(gm.w)) * den, (xb[n].w * bf16hi(gm.w)) * den);
            *(uint4*)(xs + (size_t)n * xpitch + tid * 16) = r;
        }
        consumer_sync();
}

// The consumers' half of a contraction phase: weights come out of the ring, activations from L2.
// DIRECT: the activations are not staged in shared memory; every use reads them from global memory through L1 (the
// stand-alone ring-fed contraction: a kernel of its own starts with a clean L1, and its activations were written by an
// earlier kernel, so the non-coherent path is safe there and 64 KB of them stay resident).
template <bool W4, int NT, bool DUAL, bool NORM, bool DIRECT = false, int NSLOTS = SLOTS, int SLOTB = SLOT_BYTES>
__device__ __forceinline__ bool consume_gemv(const Phase& P, const Ring& ring, uint32_t& drained, float* scratch, unsigned* gbar, int* err,
                                             unsigned long long* prof) {
    using namespace gemv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int NM = DUAL ? 2 : 1;
    constexpr int UNIT = W4 ? 64 : 32;       // k values one pass of a warp covers
    const Geom G = geom_of(W4, DUAL, P.K);
    const int units = G.stage_k / UNIT;
    // The phase's activations (norm applied) are the same for every tile: they are staged in shared memory, as a
    // whole when batch x K fits (one L2 round trip per phase), else one ring stage's K range at a time. Rows sit
    // 4 bank groups apart, like the weight rows. The inner loop reads activations from shared memory only.
    unsigned char* xs = (unsigned char*)scratch + SCRATCH_BYTES;
    const bool whole = DIRECT || (size_t)P.batch * (P.K * 2 + 64) <= (size_t)XS_BYTES;
    // k values per staged row: the whole K, else a ring stage, else (a stage of 16 rows can exceed the staging area:
    // 16 x 4096 int4 inputs are 132 KB of bf16) the largest power-of-two part of a stage that fits
    const int xspan = whole ? P.K : stage_span(P.batch, G.stage_k);
    const int xpitch = xspan * 2 + 64;
    const int units_x = xspan / UNIT;                 // units per staged span; the warps split these
    const int ux0 = (warp * units_x) / GW, ux1 = ((warp + 1) * units_x) / GW;
    const int spans_per_stage = whole ? 1 : G.stage_k / xspan;
    auto stage_x = [&](int k_begin) {
        const int cpr = xspan / 8;       // 16-byte chunks per row
        const int total = P.batch * cpr;
        // Every block stages the same bytes. Walking them from a block-dependent offset keeps the 148 blocks from asking
        // the same L2 slice for the same line at the same moment.
        const int rot = (int)(((long long)blockIdx.x * total) / gridDim.x) & ~7;
        for (int i = tid; i < total; i += CONSUMERS) {
            int idx = i + rot;
            if (idx >= total) idx -= total;
            const int n = idx / cpr, c = idx % cpr;
            const uint4 v = load_x8<NORM, true>(P.x + (size_t)n * P.K, NORM ? P.fz.norm_x + (size_t)n * P.K : nullptr, P.fz.norm_gamma,
                                                NORM ? scratch[n] : 1.0f, k_begin + c * 8, true);
            *(uint4*)(xs + (size_t)n * xpitch + c * 16) = v;
        }
    };
    if (!NORM && P.fz.ds_partial) defer_scales<true>(P.fz, P.batch, scratch);     // once per phase
    if (DIRECT) {
        // nothing to stage
    } else if (NT == 1 && NORM && P.K == CONSUMERS * 8 && P.batch <= 2) {
        stage_normed_rows(P, scratch, xs, xpitch);
    } else {
        if (NORM) row_norms<true>(P.fz, P.batch, P.K, scratch);   // once per phase
        if (whole) { stage_x(0); consumer_sync(); }
    }
    stamp(prof, 0);      // activations staged
    // this thread's activation rows (batch columns g and g + 8); a column beyond the batch reads zeros
    const bool xok0 = g < P.batch, xok1 = NT > 1 && (g + 8) < P.batch;
    const unsigned char* xs0 = DIRECT ? (const unsigned char*)(P.x + (size_t)(xok0 ? g : 0) * P.K) : xs + (size_t)(xok0 ? g : 0) * xpitch;
    const unsigned char* xs1 = DIRECT ? (const unsigned char*)(P.x + (size_t)(xok1 ? g + 8 : 0) * P.K) : xs + (size_t)(xok1 ? g + 8 : 0) * xpitch;
    auto ldx = [](const unsigned char* p) { return DIRECT ? __ldg((const uint4*)p) : *(const uint4*)p; };
    bool ok = true;
    // two sets of per-warp partial sums, used alternately, when the scratch holds them: a tile's epilogue then needs no barrier
    // against the next tile's contraction (the one barrier inside every tile's finish orders the reuse two tiles later)
    constexpr bool PINGPONG = (16 + 16 * GW + 2 * red_floats<NT, DUAL>()) * 4 <= SCRATCH_BYTES;
    int parity = 0;
    for (int gt = blockIdx.x; gt < P.n_blocks && ok; gt += gridDim.x) {
        int seg, tile;
        seg_of_tile(P.segs, P.n_segments, DUAL, gt, seg, tile);
        float acc[NM][NT][4];
#pragma unroll
        for (int mI = 0; mI < NM; ++mI)
#pragma unroll
            for (int j = 0; j < NT; ++j) acc[mI][j][0] = acc[mI][j][1] = acc[mI][j][2] = acc[mI][j][3] = 0.0f;
        // the residual this thread's epilogue will add: loaded now, so that its L2 round trip runs under the contraction
        float res_pre = 0.0f;
        const bool have_res = P.epilogue == SANIC_EPI_RESIDUAL_ADD && tid < 16 * P.batch;
        if (have_res) res_pre = __ldcg(P.residual + (size_t)(tid / 16) * P.segs.rows[0] + tile * 16 + (tid % 16));
        // int4 with stages too short to carry their scales: scale rows of fragment rows g and g+8 in global memory
        const uint16_t* sr[NM][2];
        if (W4 && G.scale_row_bytes == 0) {
#pragma unroll
            for (int mI = 0; mI < NM; ++mI) {
                const int si = DUAL ? mI : seg;
                const uint16_t* S = si == 0 ? P.segs.scales[0] : (si == 1 ? P.segs.scales[1] : P.segs.scales[2]);
                sr[mI][0] = S + (size_t)weight_row(P.epilogue, P.fz, tile, g) * (P.K / 64);
                sr[mI][1] = S + (size_t)weight_row(P.epilogue, P.fz, tile, g + 8) * (P.K / 64);
            }
        }
        for (int s = 0; s < G.n_stages; ++s, ++drained) {
            const int slot = drained % NSLOTS;
            const uint32_t parity = (drained / NSLOTS) & 1;
            const int kbase = s * G.stage_k;
            ok = mbar_wait(&ring.full[slot], parity, gbar, err, 32);
            if (!ok) break;
            const unsigned char* sb = ring.ptr + (size_t)slot * SLOTB;
            for (int sp = 0; sp < spans_per_stage; ++sp) {
            const int xbase = whole ? 0 : kbase + sp * xspan;
            if (!whole) { consumer_sync(); stage_x(xbase); consumer_sync(); }
            // this warp's units of the span (of the whole stage when everything is staged at once)
            const int u0 = whole ? (warp * units) / GW : sp * units_x + ux0;
            const int u1 = whole ? ((warp + 1) * units) / GW : sp * units_x + ux1;
#pragma unroll 2
            for (int u = u0; u < u1; ++u) {
                const int ku = u * UNIT;                 // offset inside the stage
                const int kx = kbase + ku - xbase;       // offset inside the staged activations
                if (!W4) {
                    uint4 xv[NT];
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const unsigned char* xr = j == 0 ? xs0 : xs1;
                        xv[j] = (j == 0 ? xok0 : xok1) ? ldx(xr + (size_t)(kx + t * 8) * 2) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int mI = 0; mI < NM; ++mI) {
                        const uint4 r0 = *(const uint4*)(sb + (size_t)(mI * 16 + g) * G.pitch + (ku + t * 8) * 2);
                        const uint4 r1 = *(const uint4*)(sb + (size_t)(mI * 16 + g + 8) * G.pitch + (ku + t * 8) * 2);
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            mma_bf16_16816(acc[mI][j], r0.x, r1.x, r0.y, r1.y, xv[j].x, xv[j].y);
                            mma_bf16_16816(acc[mI][j], r0.z, r1.z, r0.w, r1.w, xv[j].z, xv[j].w);
                        }
                    }
                } else {
                    const uint32_t ONES = 0x3F803F80u;
                    float sc[NM][2];
#pragma unroll
                    for (int mI = 0; mI < NM; ++mI) {
                        if (G.scale_row_bytes) {
                            sc[mI][0] = bf16_to_f32(*(const uint16_t*)(sb + G.scale_off + (size_t)(mI * 16 + g) * G.scale_row_bytes + u * 2));
                            sc[mI][1] = bf16_to_f32(*(const uint16_t*)(sb + G.scale_off + (size_t)(mI * 16 + g + 8) * G.scale_row_bytes + u * 2));
                        } else {
                            sc[mI][0] = bf16_to_f32(__ldg(sr[mI][0] + (kbase + ku) / 64));
                            sc[mI][1] = bf16_to_f32(__ldg(sr[mI][1] + (kbase + ku) / 64));
                        }
                    }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const unsigned char* xr = j == 0 ? xs0 : xs1;
                        const bool xk = j == 0 ? xok0 : xok1;
                        const uint4 xa = xk ? ldx(xr + (size_t)(kx + t * 16) * 2) : make_uint4(0, 0, 0, 0);
                        const uint4 xc = xk ? ldx(xr + (size_t)(kx + t * 16 + 8) * 2) : make_uint4(0, 0, 0, 0);
                        // activation pairs matching the nibble pairing (n_i, n_{i+4})
                        const uint32_t bA0 = prmt(xa.x, xa.z, 0x5410), bA1 = prmt(xa.x, xa.z, 0x7632);
                        const uint32_t bA2 = prmt(xa.y, xa.w, 0x5410), bA3 = prmt(xa.y, xa.w, 0x7632);
                        const uint32_t bC0 = prmt(xc.x, xc.z, 0x5410), bC1 = prmt(xc.x, xc.z, 0x7632);
                        const uint32_t bC2 = prmt(xc.y, xc.w, 0x5410), bC3 = prmt(xc.y, xc.w, 0x7632);
                        float c1[4] = {0, 0, 0, 0};
                        mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bA0, bA1);
                        mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bA2, bA3);
                        mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bC0, bC1);
                        mma_bf16_16816(c1, ONES, ONES, ONES, ONES, bC2, bC3);
#pragma unroll
                        for (int mI = 0; mI < NM; ++mI) {
                            const uint2 w0 = *(const uint2*)(sb + (size_t)(mI * 16 + g) * G.pitch + ku / 2 + t * 8);
                            const uint2 w1 = *(const uint2*)(sb + (size_t)(mI * 16 + g + 8) * G.pitch + ku / 2 + t * 8);
                            float c[4] = {0, 0, 0, 0};
                            mma_bf16_16816(c, nib_pair(w0.x), nib_pair(w1.x), nib_pair(w0.x >> 4), nib_pair(w1.x >> 4), bA0, bA1);
                            mma_bf16_16816(c, nib_pair(w0.x >> 8), nib_pair(w1.x >> 8), nib_pair(w0.x >> 12), nib_pair(w1.x >> 12), bA2, bA3);
                            mma_bf16_16816(c, nib_pair(w0.y), nib_pair(w1.y), nib_pair(w0.y >> 4), nib_pair(w1.y >> 4), bC0, bC1);
                            mma_bf16_16816(c, nib_pair(w0.y >> 8), nib_pair(w1.y >> 8), nib_pair(w0.y >> 12), nib_pair(w1.y >> 12), bC2, bC3);
                            acc[mI][j][0] = fmaf(sc[mI][0], fmaf(-136.0f, c1[0], c[0]), acc[mI][j][0]);
                            acc[mI][j][1] = fmaf(sc[mI][0], fmaf(-136.0f, c1[1], c[1]), acc[mI][j][1]);
                            acc[mI][j][2] = fmaf(sc[mI][1], fmaf(-136.0f, c1[2], c[2]), acc[mI][j][2]);
                            acc[mI][j][3] = fmaf(sc[mI][1], fmaf(-136.0f, c1[3], c[3]), acc[mI][j][3]);
                        }
                    }
                }
            }
            }   // spans of the stage
            __syncwarp();
            if (lane == 0) mbar_arrive(&ring.empty[slot]);     // this warp is done reading the slot
        }
        if (!ok) break;
        stamp(prof, 1);      // the last tile's contraction is done (overwritten per tile)
        tile_finish<NT, DUAL, true>(acc, P.batch, P.segs, P.out_dtype, P.epilogue, P.residual, P.fz, 1, 0, seg, tile, scratch, have_res, res_pre, parity);
        if (PINGPONG) parity ^= 1;
        else consumer_sync();   // the scratch is reused by the next tile
    }
    stamp(prof, 2);          // sums and epilogue done: the block is ready for the grid barrier
    return ok;
}

template <bool VT>
__device__ __forceinline__ void run_decode(const Phase& P, int per_b, unsigned char* shared, int tid, int* err) {
    for (int it = blockIdx.x; it < P.n_blocks; it += gridDim.x) {
        const int b = it / per_b, hk = (it % per_b) / P.dec.n_splits, split = it % P.dec.n_splits;
        decode::attn_decode_tile<64, VT>(P.dec, P.counters, split, hk, b, shared, tid, false, 1, err);
        decode::tile_sync(1);
    }
}

__device__ __forceinline__ void amax_merge(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}

// The producers' half of one contraction phase: this block's tiles, stage by stage, into the ring. `fill` counts the ring
// stages issued so far by all producer warps together; warp `pw` issues the stages with fill % PRODUCERS == pw.
template <int NSLOTS = SLOTS, int NPROD = PRODUCERS, int SLOTB = SLOT_BYTES>
__device__ __forceinline__ bool produce_phase(const Phase& P, const Ring& ring, uint64_t* s_full, uint64_t* s_empty, unsigned& fill, int lane,
                                              int pw, unsigned* bar, int* err) {
    bool ok = true;
    {
        const bool w4 = P.variant & 1, dual = (P.variant & 4) != 0;
        const Geom G = geom_of(w4, dual, P.K);
        const size_t full_row = w4 ? (size_t)P.K / 2 : (size_t)P.K * 2;
        const bool contiguous = w4 && G.n_stages == 1 && P.epilogue != SANIC_EPI_ROPE_CACHE;
        // The norm weight of an inlined RMSNorm is read once per step: cold in L2 by the time its phase starts
        // (gigabytes have streamed through since) and on the consumers' critical path. The producers reach the phase
        // a ring's depth early: ask L2 for it now.
        if ((P.variant & 8) && lane == 0 && pw == 0)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(P.fz.norm_gamma), "r"(P.K * 2) : "memory");
        for (int gt = blockIdx.x; gt < P.n_blocks && ok; gt += gridDim.x) {
            int seg, tile;
            seg_of_tile(P.segs, P.n_segments, dual, gt, seg, tile);
            const char* src_row = nullptr;
            const char* src_scale = nullptr;
            if (lane < G.rows) {
                const int mI = lane >> 4, r = lane & 15;
                const int si = dual ? mI : seg;
                const char* W = (const char*)(si == 0 ? P.segs.w[0] : (si == 1 ? P.segs.w[1] : P.segs.w[2]));
                const int wr = weight_row(P.epilogue, P.fz, tile, r);
                src_row = W + (size_t)wr * full_row;
                if (G.scale_row_bytes) {
                    const char* S = (const char*)(si == 0 ? P.segs.scales[0] : (si == 1 ? P.segs.scales[1] : P.segs.scales[2]));
                    src_scale = S + (size_t)wr * (P.K / 64) * 2;
                }
            }
            for (int s = 0; s < G.n_stages && ok; ++s, ++fill) {
                if ((int)(fill % NPROD) != pw) continue;
                const int slot = fill % NSLOTS;
                if (lane == 0) {
                    ok = mbar_wait(&s_empty[slot], ((fill / NSLOTS) & 1) ^ 1, bar, err, 33);
                    if (ok) mbar_expect_tx(&s_full[slot], (uint32_t)(G.rows * (G.row_bytes + G.scale_row_bytes)));
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (contiguous) {
                    // whole rows, 16 consecutive ones per matrix: one copy of the weights and one of the scales per matrix
                    if (ok && lane < G.rows && (lane & 15) == 0) {
                        bulk_load(ring.base + slot * SLOTB + lane * G.pitch, src_row, (uint32_t)(16 * G.row_bytes), &s_full[slot]);
                        if (G.scale_row_bytes)
                            bulk_load(ring.base + slot * SLOTB + G.scale_off + lane * G.scale_row_bytes, src_scale,
                                      (uint32_t)(16 * G.scale_row_bytes), &s_full[slot]);
                    }
                } else if (ok && lane < G.rows) {
                    bulk_load(ring.base + slot * SLOTB + lane * G.pitch, src_row + (size_t)s * G.row_bytes, (uint32_t)G.row_bytes, &s_full[slot]);
                    if (G.scale_row_bytes)
                        bulk_load(ring.base + slot * SLOTB + G.scale_off + lane * G.scale_row_bytes,
                                  src_scale + (size_t)s * G.scale_row_bytes, (uint32_t)G.scale_row_bytes, &s_full[slot]);
                }
            }
        }
    }
    return ok;
}

// One instantiation per batch width (a program's contractions share it): fewer bodies per kernel keep the
// register allocation of each one clean. Weight storage may differ per stage (int4 layers, bf16 lm_head);
// ANY_I4 = false leaves the int4 bodies out for programs that have none.
template <int NT, bool ANY_I4>
__global__ void __launch_bounds__(THREADS, 1)
decode_step_kernel(const Phase* __restrict__ phases, int n_phases, unsigned* bar, int* err, unsigned long long* stamps,
                   unsigned long long* prof) {
    extern __shared__ __align__(128) unsigned char dyn[];       // [weight ring][shared region]
    __shared__ Phase ph[2];
    __shared__ __align__(8) uint64_t s_full[SLOTS], s_empty[SLOTS];
    __shared__ int s_ok;
    __shared__ unsigned s_produced;
    const int tid = threadIdx.x;
    unsigned char* shared = dyn + RING_BYTES;
    Ring ring{s_full, s_empty, smem_u32(dyn), dyn};
    if (tid == 0) {
        for (int i = 0; i < SLOTS; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], gemv::GW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_produced = 0;
    }
    constexpr int PW = sizeof(Phase) / 4;
    if (tid < CONSUMERS)
        for (int w = tid; w < PW; w += CONSUMERS) ((int*)&ph[0])[w] = __ldg((const int*)&phases[0] + w);
    __syncthreads();

    if (tid >= CONSUMERS) {
        // ── producer warp: streams the weights of every contraction phase, in the order the consumers will want
        //    them, as far ahead as the ring allows. Weights never change, so it may run ahead of the grid barriers;
        //    HBM keeps streaming while the consumers wait for activations. ──
        const int lane = tid & 31, pw = (tid - CONSUMERS) >> 5;
        unsigned fill = 0;
        bool ok = true;
        for (int i = 0; i < n_phases && ok; ++i) {
            const Phase& P = phases[i];
            if (P.op != PH_GEMV) continue;
            ok = produce_phase(P, ring, s_full, s_empty, fill, lane, pw, bar, err);
        }
        if (lane == 0 && pw == 0) s_produced = fill;
    } else {
        // ── consumers: walk the phases ──
        uint32_t drained = 0;
        bool ok = true;
        if (blockIdx.x == 0 && tid == 0) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); stamps[0] = g; }
        for (int i = 0; i < n_phases && ok; ++i) {
            const Phase& P = ph[i & 1];
            // The next descriptor: the table is cold in L2 (it is read once per step), so its load is issued now, into a
            // register, and stored to shared memory only when the phase body is done: the miss runs under the phase.
            static_assert(PW <= CONSUMERS, "one descriptor word per consumer thread");
            int next_word = 0;
            if (i + 1 < n_phases && tid < PW) next_word = __ldg((const int*)&phases[i + 1] + tid);
            switch (P.op) {
                case PH_GEMV: {
                    float* scratch = (float*)shared;
                    switch (((P.variant >> 1) & 6) | (P.variant & 1)) {      // bit0: int4, bit1: silu-mul pair, bit2: inlined norm
                        case 0: ok = consume_gemv<false, NT, false, false>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 1: if (ANY_I4) ok = consume_gemv<true, NT, false, false>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 2: ok = consume_gemv<false, NT, true, false>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 3: if (ANY_I4) ok = consume_gemv<true, NT, true, false>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 4: ok = consume_gemv<false, NT, false, true>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 5: if (ANY_I4) ok = consume_gemv<true, NT, false, true>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 6: ok = consume_gemv<false, NT, true, true>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                        case 7: if (ANY_I4) ok = consume_gemv<true, NT, true, true>(P, ring, drained, scratch, bar, err, prof ? prof + 3 * i : nullptr); break;
                    }
                    break;
                }
                case PH_DECODE: {
                    // one item = (chunk, kv head, batch) on the first 128 threads; its K/V ring is the shared region
                    const int per_b = P.dec.n_splits * P.dec.kv_heads;
                    if (tid < 128) {
                        if (P.variant & 1) run_decode<true>(P, per_b, shared, tid, err);
                        else run_decode<false>(P, per_b, shared, tid, err);
                    }
                    break;
                }
                case PH_EMBED: {   // out[b,:] = widen(table[token[b],:]); variant 1: int4 nibbles times the group scale
                    const int32_t* tokens = (const int32_t*)P.b;
                    float* out = (float*)P.c;
                    const int hidden = P.i1, vocab = P.i2;
                    for (int b = blockIdx.x; b < P.n_blocks; b += gridDim.x) {
                        int tok = __ldcg(tokens + b);
                        tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
                        if (P.variant & 1) {
                            const uint8_t* row = (const uint8_t*)P.a + (size_t)tok * (hidden / 2);
                            const uint16_t* srow = (const uint16_t*)P.scratch + (size_t)tok * (hidden / P.i0);
                            for (int k = tid; k < hidden; k += CONSUMERS)
                                out[(size_t)b * hidden + k] = (float)(((row[k >> 1] >> ((k & 1) * 4)) & 0xF) - 8) * bf16_to_f32(srow[k / P.i0]);
                        } else {
                            const uint16_t* table = (const uint16_t*)P.a;
                            for (int k = tid; k < hidden; k += CONSUMERS) out[(size_t)b * hidden + k] = bf16_to_f32(table[(size_t)tok * hidden + k]);
                        }
                    }
                    break;
                }
                case PH_RMSNORM: {   // xn = bf16((x * g) / sqrt(sum(x^2) * (1/n) + eps)), fixed summation order
                    const float* x = (const float*)P.a;
                    const uint16_t* gamma = (const uint16_t*)P.b;
                    uint16_t* out = (uint16_t*)P.c;
                    const int n = P.i1;
                    float* wsum = (float*)shared;
                    for (int row = blockIdx.x; row < P.n_blocks; row += gridDim.x) {
                        const float* xr = x + (size_t)row * n;
                        float ss = 0.0f;
                        for (int k = tid; k < n; k += CONSUMERS) { const float v = __ldcg(xr + k); ss = fmaf(v, v, ss); }
                        ss = warp_sum(ss);
                        if ((tid & 31) == 0) wsum[tid >> 5] = ss;
                        consumer_sync();
                        if (tid == 0) {
                            float tot = 0.0f;
                            for (int w = 0; w < 8; ++w) tot += wsum[w];
                            wsum[8] = sqrtf(tot * (1.0f / (float)n) + P.f0);
                        }
                        consumer_sync();
                        const float den = wsum[8];
                        for (int k = tid; k < n; k += CONSUMERS)
                            out[(size_t)row * n + k] = f32_to_bf16_bits((__ldcg(xr + k) * bf16_to_f32(gamma[k])) / den);
                        consumer_sync();
                    }
                    break;
                }
                case PH_ARGMAX_PART: {   // (max value, first index) per chunk of a row
                    const float* x = (const float*)P.a;
                    const int n = P.i1;
                    float* sv = (float*)shared; int* si = (int*)shared + 8;
                    for (int blk = blockIdx.x; blk < P.n_blocks; blk += gridDim.x) {
                        const int row = blk / AMAX_CHUNKS, chunk = blk % AMAX_CHUNKS;
                        const int lo = (int)(((long long)chunk * n) / AMAX_CHUNKS), hi = (int)(((long long)(chunk + 1) * n) / AMAX_CHUNKS);
                        const float* xr = x + (size_t)row * n;
                        float v = -INFINITY; int idx = 0x7FFFFFFF;
                        for (int j = lo + tid; j < hi; j += CONSUMERS) amax_merge(v, idx, __ldcg(xr + j), j);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            float v2 = __shfl_xor_sync(0xffffffffu, v, o); int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
                            amax_merge(v, idx, v2, i2);
                        }
                        if ((tid & 31) == 0) { sv[tid >> 5] = v; si[tid >> 5] = idx; }
                        consumer_sync();
                        if (tid == 0) {
                            for (int w = 1; w < 8; ++w) amax_merge(v, idx, sv[w], si[w]);
                            P.scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2] = v;
                            P.scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2 + 1] = __int_as_float(idx);
                        }
                        consumer_sync();
                    }
                    break;
                }
                case PH_ARGMAX_FINAL: {
                    uint32_t* out = (uint32_t*)P.c;
                    float* sv = (float*)shared; int* si = (int*)shared + 8;
                    for (int row = blockIdx.x; row < P.n_blocks; row += gridDim.x) {
                        float v = -INFINITY; int idx = 0x7FFFFFFF;
                        if (tid < AMAX_CHUNKS) {
                            v = __ldcg(P.scratch + ((size_t)row * AMAX_CHUNKS + tid) * 2);
                            idx = __float_as_int(__ldcg(P.scratch + ((size_t)row * AMAX_CHUNKS + tid) * 2 + 1));
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            float v2 = __shfl_xor_sync(0xffffffffu, v, o); int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
                            amax_merge(v, idx, v2, i2);
                        }
                        if ((tid & 31) == 0) { sv[tid >> 5] = v; si[tid >> 5] = idx; }
                        consumer_sync();
                        if (tid == 0) {
                            for (int w = 1; w < 8; ++w) amax_merge(v, idx, sv[w], si[w]);
                            out[row] = (idx == 0x7FFFFFFF) ? 0xFFFFFFFFu : (uint32_t)idx;   // the +inf identity saturates to u32::MAX
                        }
                        consumer_sync();
                    }
                    break;
                }
                case PH_ADVANCE:
                    if (blockIdx.x == 0 && tid == 0) *(int32_t*)P.c += 1;
                    break;
                default: break;
            }
            if (i + 1 < n_phases && tid < PW) ((int*)&ph[(i + 1) & 1])[tid] = next_word;     // visible after the barrier's block syncs
            if (ok && i + 1 < n_phases) ok = grid_barrier(bar, (unsigned)(i + 1) * gridDim.x, err, &s_ok);
            if (blockIdx.x == 0 && tid == 0) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); stamps[i + 1] = g; }
        }
        if (!ok && tid == 0) atomicExch(bar + 1, 1u);      // make sure the producer stops too
    }
    // Leave only when no copy into this CTA's shared memory is still in flight: after the producer has stopped,
    // thread 0 waits (bounded) for every stage that was issued, consumed or not.
    __syncthreads();
    if (tid == 0) {
        const unsigned produced = s_produced;
        const unsigned first = produced > SLOTS ? produced - SLOTS : 0;
        for (unsigned f = first; f < produced; ++f) {
            bool done = false;
            for (unsigned it = 0; it < SPIN_LIMIT && !done; ++it) done = mbar_test(&s_full[f % SLOTS], (f / SLOTS) & 1);
        }
    }
    __syncthreads();
}

// One contraction as a kernel of its own, fed like a phase of the step kernel: producer warps stream the weights through
// the shared-memory ring with bulk copies, consumer warps take their activations from global memory through L1. Used by
// the launch-list form at batch > 8, where the register-staged loads of gemv_mma_kernel (two 64-blocks per warp: what 128
// registers hold beside two accumulator tiles) keep about 10 MB in flight and 19 MB saturate HBM; the ring holds
// 64 KB per block in flight whatever the consumers' registers do. bf16: two slots and two blocks per SM (90 KB of shared
// memory and at most 112 registers each), so that the blocks of the NEXT kernel of a launch list become resident while
// this one drains and their producers stream weights through the kernel boundary; int4 needs more registers than two
// blocks per SM leave and runs four slots, one block per SM. The weights do not depend on the stream predecessor,
// so the producers start before the programmatic-launch wait; the consumers wait before they touch activations.
template <bool W4, bool DUAL, int NSLOTS, int SLOTB, int PER_SM>
__global__ void __launch_bounds__(RING_THREADS, PER_SM) gemv_ring_kernel(const __grid_constant__ Phase P, int* err) {
    extern __shared__ __align__(128) unsigned char dyn[];       // [weight ring][contraction scratch]
    __shared__ __align__(8) uint64_t s_full[NSLOTS], s_empty[NSLOTS];
    __shared__ unsigned s_produced;
    const int tid = threadIdx.x;
    Ring ring{s_full, s_empty, smem_u32(dyn), dyn};
    if (tid == 0) {
        for (int i = 0; i < NSLOTS; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], gemv::GW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_produced = 0;
    }
    __syncthreads();
    if (tid >= CONSUMERS) {
        // one producer warp: a stage is 16 or 32 row copies issued by as many lanes
        const int lane = tid & 31;
        unsigned fill = 0;
        produce_phase<NSLOTS, 1, SLOTB>(P, ring, s_full, s_empty, fill, lane, 0, nullptr, err);
        if (lane == 0) s_produced = fill;
    } else {
        griddep_launch();
        griddep_wait();
        uint32_t drained = 0;
        consume_gemv<W4, 2, DUAL, false, true, NSLOTS, SLOTB>(P, ring, drained, (float*)(dyn + NSLOTS * SLOTB), nullptr, err, nullptr);
    }
    __syncthreads();
    if (tid == 0) {      // no copy into this CTA's shared memory may still be in flight when it exits
        const unsigned produced = s_produced;
        const unsigned first = produced > (unsigned)NSLOTS ? produced - NSLOTS : 0;
        for (unsigned f = first; f < produced; ++f) {
            bool done = false;
            for (unsigned it = 0; it < SPIN_LIMIT && !done; ++it) done = mbar_test(&s_full[f % NSLOTS], (f / NSLOTS) & 1);
        }
    }
    __syncthreads();
}

}  // namespace

struct Plan {
    const void* kernel = nullptr;
    Phase* d_phases = nullptr;
    unsigned* d_bar = nullptr;
    unsigned long long* d_stamps = nullptr;
    unsigned long long* d_prof = nullptr;     // 3 stamps per phase, taken by block 0 inside contraction phases
    int n = 0;
    int grid = 0;
    size_t smem = 0;
};

int phases(const Plan* plan) { return plan ? plan->n : 0; }

void destroy(Plan* plan) {
    if (!plan) return;
    if (plan->d_phases) cudaFree(plan->d_phases);
    if (plan->d_bar) cudaFree(plan->d_bar);
    if (plan->d_stamps) cudaFree(plan->d_stamps);
    if (plan->d_prof) cudaFree(plan->d_prof);
    delete plan;
}

// The ring-fed contraction for one stage of a launch list (batch > 8, no inlined norm). SANIC_ERR_UNSUPPORTED when the shape
// has no ring geometry; the caller then uses the register-staged kernel.
int32_t gemv_ring(sanic_ctx* ctx, const sanic_gemv_params* g, cudaStream_t stream) {
    Phase P{};
    int tiles = 0;
    int32_t rc = gemv::host_prepare(ctx, g, P.segs, P.fz, tiles);
    if (rc != SANIC_OK) return rc;
    const bool w4 = g->weight_dtype == SANIC_I4, dual = g->epilogue == SANIC_EPI_SILU_MUL;
    if (g->batch <= 8 || g->norm_x) return SANIC_ERR_UNSUPPORTED;
    const Geom G = geom_of(w4, dual, g->K);
    if (G.stage_k < 256 || g->K % G.stage_k != 0) return SANIC_ERR_UNSUPPORTED;
    P.op = PH_GEMV; P.n_blocks = tiles;
    P.variant = (w4 ? 1 : 0) | 2 | (dual ? 4 : 0);
    P.x = (const uint16_t*)g->x; P.batch = g->batch; P.K = g->K; P.n_segments = g->n_segments;
    P.out_dtype = g->out_dtype; P.epilogue = g->epilogue; P.residual = g->residual;
    sanic_set_device(ctx);
    auto go = [&](auto kern, int slots, int slot_bytes, int scratch_bytes, int per_sm) -> int32_t {
        const size_t smem = (size_t)slots * slot_bytes + scratch_bytes;
        SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // every block must be resident at once: the programmatic launch of the next kernel may only follow blocks that
        // have started, and blocks of that kernel then hold SM slots until this one has finished
        cudaError_t e = launch_pdl(kern, dim3(std::min(tiles, per_sm * ctx->sm_count)), dim3(RING_THREADS), smem, stream, P, ctx->status_dev);
        if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemv (ring): ") + cudaGetErrorString(e));
        return SANIC_OK;
    };
    if (w4) return dual ? go(gemv_ring_kernel<true, true, 4, SLOT_BYTES, 1>, 4, SLOT_BYTES, SCRATCH_BYTES, 1)
                        : go(gemv_ring_kernel<true, false, 4, SLOT_BYTES, 1>, 4, SLOT_BYTES, SCRATCH_BYTES, 1);
    // bf16. More tiles than SMs: two slots, two blocks per SM (90 KB each). At most one tile per SM: three slots keep the bytes
    // in flight up, and their 125 KB still leave room for a two-slot block of the next kernel beside them. (Three slots of
    // exactly a stage's size, two blocks per SM, measured slower: 1.06 against 1.03 ms per step at batch 16.)
    if (tiles <= ctx->sm_count)
        return dual ? go(gemv_ring_kernel<false, true, 3, SLOT_BYTES, 2>, 3, SLOT_BYTES, SCRATCH_BYTES, 1)
                    : go(gemv_ring_kernel<false, false, 3, SLOT_BYTES, 2>, 3, SLOT_BYTES, SCRATCH_BYTES, 1);
    return dual ? go(gemv_ring_kernel<false, true, 2, SLOT_BYTES, 2>, 2, SLOT_BYTES, SCRATCH_BYTES, 2)
                : go(gemv_ring_kernel<false, false, 2, SLOT_BYTES, 2>, 2, SLOT_BYTES, SCRATCH_BYTES, 2);
}

int32_t build(sanic_ctx* ctx, const std::vector<sanic_stage_desc>& stages, Plan** out) {
    *out = nullptr;
    std::vector<Phase> ph;
    int group = -1;      // 1: batch > 8, shared by every contraction of the program
    bool any_i4 = false;
    for (const sanic_stage_desc& s : stages) {
        Phase P{};
        switch (s.op) {
            case SANIC_OP_GEMV: {
                const sanic_gemv_params& g = s.u.gemv;
                int tiles = 0;
                int32_t rc = gemv::host_prepare(ctx, &g, P.segs, P.fz, tiles);
                if (rc != SANIC_OK) return rc;
                const bool w4 = g.weight_dtype == SANIC_I4, wide = g.batch > 8, dual = g.epilogue == SANIC_EPI_SILU_MUL,
                           norm = g.norm_x != nullptr;
                if (group >= 0 && group != (wide ? 1 : 0)) return SANIC_ERR_UNSUPPORTED;
                group = wide ? 1 : 0;
                any_i4 = any_i4 || w4;
                {   // a ring stage must give every warp at least one pass
                    const Geom G = geom_of(w4, dual, g.K);
                    if (G.stage_k < 256 || g.K % G.stage_k != 0) return SANIC_ERR_UNSUPPORTED;
                }
                P.op = PH_GEMV; P.n_blocks = tiles;
                P.variant = (w4 ? 1 : 0) | (wide ? 2 : 0) | (dual ? 4 : 0) | (norm ? 8 : 0);
                P.x = (const uint16_t*)g.x; P.batch = g.batch; P.K = g.K; P.n_segments = g.n_segments;
                P.out_dtype = g.out_dtype; P.epilogue = g.epilogue; P.residual = g.residual;
                break;
            }
            case SANIC_OP_DECODE_ATTN: {
                const sanic_decode_params& d = s.u.decode;
                int32_t rc = decode::host_validate(ctx, &d);
                if (rc != SANIC_OK) return rc;
                P.op = PH_DECODE; P.dec = d;
                P.n_blocks = d.n_splits * d.kv_heads * d.batch;
                // head_dim 128 keeps 64 more accumulator registers per thread than this kernel's budget of 128 holds
                if (d.head_dim != 64) return SANIC_ERR_UNSUPPORTED;
                P.variant = d.v_transposed ? 1 : 0;
                P.counters = (int*)(d.partials + (size_t)d.batch * d.q_heads * d.n_splits * (d.head_dim + 2));
                break;
            }
            case SANIC_OP_EMBED:
                SANIC_REQUIRE(ctx, s.u.embed.table && s.u.embed.tokens && s.u.embed.out && s.u.embed.batch > 0, "step: bad embed stage");
                P.op = PH_EMBED; P.n_blocks = s.u.embed.batch;
                P.a = s.u.embed.table; P.b = s.u.embed.tokens; P.c = s.u.embed.out; P.i1 = s.u.embed.hidden; P.i2 = s.u.embed.vocab;
                if (s.u.embed.table_dtype == SANIC_I4) {
                    SANIC_REQUIRE(ctx, s.u.embed.scales && s.u.embed.group > 0 && s.u.embed.group % 2 == 0 && s.u.embed.hidden % s.u.embed.group == 0,
                                  "step: an int4 embed stage needs scales and an even group size dividing hidden");
                    P.variant = 1; P.i0 = s.u.embed.group; P.scratch = (float*)s.u.embed.scales;
                }
                break;
            case SANIC_OP_RMSNORM:
                SANIC_REQUIRE(ctx, s.u.rmsnorm.x && s.u.rmsnorm.gamma && s.u.rmsnorm.out && s.u.rmsnorm.rows > 0 && s.u.rmsnorm.n > 0,
                              "step: bad rmsnorm stage");
                P.op = PH_RMSNORM; P.n_blocks = s.u.rmsnorm.rows;
                P.a = s.u.rmsnorm.x; P.b = s.u.rmsnorm.gamma; P.c = s.u.rmsnorm.out; P.i1 = s.u.rmsnorm.n; P.f0 = s.u.rmsnorm.eps;
                break;
            case SANIC_OP_ARGMAX: {
                SANIC_REQUIRE(ctx, s.u.argmax.x && s.u.argmax.out && s.u.argmax.scratch && s.u.argmax.rows > 0 && s.u.argmax.n > 0,
                              "step: bad argmax stage");
                P.op = PH_ARGMAX_PART; P.n_blocks = s.u.argmax.rows * AMAX_CHUNKS;
                P.a = s.u.argmax.x; P.i1 = s.u.argmax.n; P.scratch = s.u.argmax.scratch;
                ph.push_back(P);
                P = Phase{};
                P.op = PH_ARGMAX_FINAL; P.n_blocks = s.u.argmax.rows; P.c = s.u.argmax.out; P.scratch = s.u.argmax.scratch;
                break;
            }
            case SANIC_OP_ADVANCE:
                SANIC_REQUIRE(ctx, s.u.advance.position, "step: bad advance stage");
                P.op = PH_ADVANCE; P.n_blocks = 1; P.c = s.u.advance.position;
                break;
            default:
                return SANIC_ERR_UNSUPPORTED;
        }
        ph.push_back(P);
    }
    static_assert(gemv::scratch_floats<2, true>() * 4 <= SCRATCH_BYTES && decode::Cfg<64>::SMEM <= SHARED_BYTES, "shared region too small");
    const size_t smem = RING_BYTES + SHARED_BYTES;
    sanic_set_device(ctx);
    const void* kernel = group == 1 ? (any_i4 ? (const void*)decode_step_kernel<2, true> : (const void*)decode_step_kernel<2, false>)
                                    : (any_i4 ? (const void*)decode_step_kernel<1, true> : (const void*)decode_step_kernel<1, false>);
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    SANIC_CUDA_CHECK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem));
    if (per_sm < 1) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "step: the persistent kernel does not fit on an SM");
    int coop = 0;
    SANIC_CUDA_CHECK(ctx, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    if (!coop) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "step: the device has no cooperative launch");
    Plan* plan = new (std::nothrow) Plan();
    if (!plan) return SANIC_ERR_NOMEM;
    plan->n = (int)ph.size();
    plan->kernel = kernel;
    plan->grid = ctx->sm_count;     // one block per SM: each phase body may use the whole register file
    plan->smem = smem;
    cudaError_t e = cudaMalloc(&plan->d_phases, ph.size() * sizeof(Phase));
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_bar, 2 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_stamps, (ph.size() + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(plan->d_stamps, 0, (ph.size() + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_prof, 3 * ph.size() * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(plan->d_prof, 0, 3 * ph.size() * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemcpy(plan->d_phases, ph.data(), ph.size() * sizeof(Phase), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { destroy(plan); return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("step: ") + cudaGetErrorString(e)); }
    *out = plan;
    return SANIC_OK;
}

int32_t launch(sanic_ctx* ctx, Plan* plan, cudaStream_t stream) {
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaMemsetAsync(plan->d_bar, 0, 2 * sizeof(unsigned), stream));
    const Phase* phases_arg = plan->d_phases;
    int n = plan->n;
    unsigned* bar = plan->d_bar;
    int* err = ctx->status_dev;
    unsigned long long* stamps = plan->d_stamps;
    unsigned long long* prof = plan->d_prof;
    void* args[] = {(void*)&phases_arg, (void*)&n, (void*)&bar, (void*)&err, (void*)&stamps, (void*)&prof};
    cudaError_t e = cudaLaunchCooperativeKernel(plan->kernel, dim3(plan->grid), dim3(THREADS), args, plan->smem, stream);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("step: ") + cudaGetErrorString(e));
    return SANIC_OK;
}

// Seconds each phase of the last completed step took on the device (the caller has synchronised). For the last
// phase the interval ends when CTA 0 leaves it; earlier phases end at the barrier, i.e. include waiting for the
// slowest CTA. Returns the number of phases written.
int32_t phase_times(sanic_ctx* ctx, Plan* plan, double* seconds, int cap) {
    std::vector<unsigned long long> h(plan->n + 1);
    SANIC_CUDA_CHECK(ctx, cudaMemcpy(h.data(), plan->d_stamps, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    int n = std::min(cap, plan->n);
    for (int i = 0; i < n; ++i) seconds[i] = (double)(h[i + 1] - h[i]) * 1e-9;
    return n;
}

// The same step in finer grain, for contraction phases (block 0's view): seconds from the phase's start to its
// activations being staged, to the end of its last tile's contraction, to the end of its sums and epilogue, and to the
// release of the grid barrier that ends it. Four numbers per phase; a phase that is not a contraction reports 0, 0, 0
// and its whole time. Returns the number of phases written.
int32_t phase_profile(sanic_ctx* ctx, Plan* plan, double* out, int cap) {
    std::vector<unsigned long long> h(plan->n + 1), pr(3 * (size_t)plan->n);
    SANIC_CUDA_CHECK(ctx, cudaMemcpy(h.data(), plan->d_stamps, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    SANIC_CUDA_CHECK(ctx, cudaMemcpy(pr.data(), plan->d_prof, pr.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    int n = std::min(cap, plan->n);
    for (int i = 0; i < n; ++i) {
        for (int k = 0; k < 3; ++k) {
            const unsigned long long t = pr[3 * (size_t)i + k];
            out[4 * i + k] = (t >= h[i] && t <= h[i + 1]) ? (double)(t - h[i]) * 1e-9 : 0.0;
        }
        out[4 * i + 3] = (double)(h[i + 1] - h[i]) * 1e-9;
    }
    return n;
}

}  // namespace step
}  // namespace sanic
