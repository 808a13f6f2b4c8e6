// Deferred-normaliser contraction (RMSNorm-fused GEMM) on the 5th-generation tensor cores.
//
//   y[i,j] = (sum_k x[i,k] * g[k] * W[k,j]) / sqrt(sum_k x[i,k]^2 / K + eps)
//
// The derived carrier has two Plain(Add) slots over the same K stream and a project that
// divides once at the end (reference tests/laws.rs:620-646, src/partition.rs:2591-2608), so
// the main loop is a plain tensor-core GEMM on A' = bf16(x * g) and the epilogue scales each
// row by 1/sqrt(.). The fusion lives in the prologue of each K stage: a transform warpgroup reads
// the A tile that TMA brought into shared memory, multiplies by g, accumulates sum x^2 per row from
// the same bytes, and hands the tile to the tensor core THROUGH TENSOR MEMORY (the MMA takes its A
// operand from TMEM). x is read from HBM exactly once, and shared memory carries each operand byte
// once in and once out: rewriting A in place instead cost 32 KB more shared-memory traffic per k-block,
// and shared-memory bandwidth is what bounds a one-CTA 128x256 tile.
//
// Persistent kernel, one CTA per SM, 128x256 output tile, BK = 64, 4-stage TMA ring.
//   warp 0      TMA producer (cp.async.bulk.tensor, 128B swizzle, mbarrier complete_tx)
//   warp 1      MMA issuer (tcgen05.mma cta_group::1 kind::f16, A from TMEM, M=128 N=256 K=16 per instruction)
//   warp 2      TMEM allocator (256 accumulator columns + 4 x 32 columns of A stages)
//   warps 4-11  A transform: shared memory -> x*g -> TMEM, + sum x^2 (two threads per row)
//   warps 12-15 epilogue: tcgen05.ld, * rsqrt, bf16/f32 stores
// Every mbarrier wait is bounded; on expiry the kernel records an error code in the context's
// status word, drains and frees its TMEM, and the next sanic_sync returns SANIC_ERR_TIMEOUT.
//
// Roofline: tensor-bound. FLOPs = 2*M*N*K; HBM bytes = x + W + y (about 117 MB at
// 4096x2048x8192, 61 us at 2.25 PFLOP/s).
#include <cuda.h>
#include <cstdio>

#include "common.cuh"

namespace {
using namespace sanic;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int MAX_K = 8192;
constexpr int NTHREADS = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr uint32_t P_SPIN_LIMIT = 1u << 22;   // the pair kernel: waits that cross CTAs, kept short
constexpr int TM_A = BN;                      // tensor-memory columns: [0, BN) accumulator, then STAGES x 32 columns of A

struct Shared {
    uint64_t full[STAGES], ready[STAGES], empty[STAGES];
    uint64_t tmem_full, tmem_empty, ss_full[2], ss_empty[2];
    uint32_t tmem_base;
    volatile int abort_flag;
    float ss[2][2][BM];   // [accumulator slot][row half][row]
};

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait. Returns false if the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Shared* sh, int* err, int code) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u && sh->abort_flag) return false;
    }
    sh->abort_flag = 1;
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory: lane = row, each 32-bit column holds two consecutive K
// elements, so one K=16 step reads 8 columns starting at a_tmem.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 16 columns: thread i of the warp writes 16 consecutive columns of lane (base lane + i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (128B swizzle). lbo / sbo in bytes.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version of this architecture
    d |= (uint64_t)2 << 61;   // SWIZZLE_128B
    return d;
}

struct Pipe {
    int stage = 0;
    uint32_t phase = 0;
    __device__ void advance() { if (++stage == STAGES) { stage = 0; phase ^= 1; } }
};

__global__ void __launch_bounds__(NTHREADS, 1)
gemm_rmsnorm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const uint16_t* __restrict__ gamma, void* __restrict__ y, int M, int N, int K, int w_is_nk,
                    float eps, int out_dtype, int* err) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;              // swizzle atoms need 1024-byte alignment
    unsigned char* aligned = smem_dyn + (base - raw);
    uint16_t* gsm = (uint16_t*)(aligned + STAGES * STAGE_BYTES);  // gamma, padded to a multiple of BK
    Shared* sh = (Shared*)(aligned + STAGES * STAGE_BYTES + MAX_K * 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (K + BK - 1) / BK;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->ready[s], 8); mbar_init(&sh->empty[s], 1); }
        mbar_init(&sh->tmem_full, 1); mbar_init(&sh->tmem_empty, 4);
        for (int a = 0; a < 2; ++a) { mbar_init(&sh->ss_full[a], 8); mbar_init(&sh->ss_empty[a], 4); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < kblocks * BK; i += NTHREADS) gsm[i] = (i < K) ? gamma[i] : (uint16_t)0;
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ── TMA producer ──
        if (lane == 0) {
            Pipe p; p.phase = 1;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
                const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(&sh->empty[p.stage], p.phase, sh, err, 1);
                    if (!ok) break;
                    const uint32_t sa = base + p.stage * STAGE_BYTES, sb = sa + A_BYTES;
                    mbar_expect_tx(&sh->full[p.stage], STAGE_BYTES);
                    tma_load_2d(sa, &map_a, &sh->full[p.stage], kb * BK, m0);
                    if (w_is_nk) {
                        tma_load_2d(sb, &map_b, &sh->full[p.stage], kb * BK, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * (64 * BK * 2), &map_b, &sh->full[p.stage], n0 + 64 * j, kb * BK);
                    }
                    p.advance();
                }
            }
        }
    } else if (warp == 1) {
        // ── MMA issuer ──
        if (lane == 0) {
            // instruction descriptor: D f32, A/B bf16, A K-major, B K- or MN-major, N=256, M=128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((w_is_nk ? 0u : 1u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            Pipe p;
            int use = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++use) {
                ok = mbar_wait(&sh->tmem_empty, (use & 1) ^ 1, sh, err, 2);     // the epilogue has read the previous tile
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(&sh->ready[p.stage], p.phase, sh, err, 3);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sb = base + p.stage * STAGE_BYTES + A_BYTES;
                    const uint32_t a_tmem = tmem + TM_A + p.stage * (BK / 2);
                    const uint64_t bdesc = w_is_nk ? make_desc(sb, 16, 1024) : make_desc(sb, 64 * BK * 2, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // A: 16 elements = 8 tensor-memory columns; B K-major: 32 bytes along the swizzled row; MN-major: 16 k-rows = 2048 bytes
                        const uint64_t bd = bdesc + (uint64_t)(w_is_nk ? k * 2 : k * 128);
                        umma_f16_ts(acc, a_tmem + 8 * k, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&sh->empty[p.stage]);      // stage reusable once these MMAs have read it
                    p.advance();
                }
                if (ok) umma_commit(&sh->tmem_full);
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ── A transform: shared memory -> x*g -> tensor memory, sum x^2 ──
        const int idx = threadIdx.x - 128;
        const int row = idx & (BM - 1), half = idx >> 7;   // half 0: chunks 0-3, half 1: chunks 4-7
        // this warp may touch tensor-memory lanes 32*(warp%4)..+31, which are exactly its rows
        const uint32_t a_lane = tmem + ((uint32_t)(row & ~31) << 16) + TM_A + half * (BK / 4);
        Pipe p;
        int use = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++use) {
            const int a = use & 1;
            float ss = 0.0f;
            for (int kb = 0; kb < kblocks; ++kb) {
                ok = mbar_wait(&sh->full[p.stage], p.phase, sh, err, 4);
                if (!ok) break;
                const unsigned char* arow = aligned + p.stage * STAGE_BYTES + row * 128;
                uint32_t av[16];
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int c = half * 4 + c4;
                    const uint4 v = *(const uint4*)(arow + ((c ^ (row & 7)) << 4));
                    const uint4 gv = *(const uint4*)(gsm + kb * BK + c * 8);
                    uint32_t xs[4] = {v.x, v.y, v.z, v.w};
                    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float x0 = bf16lo(xs[j]), x1 = bf16hi(xs[j]);
                        ss = fmaf(x0, x0, ss); ss = fmaf(x1, x1, ss);
                        // bf16 x bf16 is exact in f32, so the packed bf16 multiply (round to nearest even
                        // of the exact product) equals bf16(float(x) * float(g)) bit for bit
                        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(xs[j]) : "r"(xs[j]), "r"(gs[j]));
                    }
                    av[4 * c4] = xs[0]; av[4 * c4 + 1] = xs[1]; av[4 * c4 + 2] = xs[2]; av[4 * c4 + 3] = xs[3];
                }
                // 32 k values = 16 columns of this row's lane in the stage's A slot (free: the stage's previous MMAs
                // retired before the producer refilled the stage this thread just read)
                tmem_st16(a_lane + p.stage * (BK / 2), av);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->ready[p.stage]);
                p.advance();
            }
            if (!ok) break;
            ok = mbar_wait(&sh->ss_empty[a], ((use >> 1) & 1) ^ 1, sh, err, 5);
            if (!ok) break;
            sh->ss[a][half][row] = ss;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->ss_full[a]);
        }
    } else if (warp >= 12) {
        // ── epilogue ──
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        const bool wide_ok = (N % 16 == 0) && (((uintptr_t)y & 31) == 0);     // 32-byte stores need 32-byte aligned rows
        int use = 0;
        bool ok = true;
        const float inv_k = 1.0f / (float)K;
        for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++use) {
            const int a = use & 1;
            const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
            ok = mbar_wait(&sh->ss_full[a], (use >> 1) & 1, sh, err, 6);
            if (!ok) break;
            const float ssv = sh->ss[a][0][row] + sh->ss[a][1][row];
            const float rstd = 1.0f / sqrtf(ssv * inv_k + eps);
            ok = mbar_wait(&sh->tmem_full, use & 1, sh, err, 7);
            if (!ok) break;
            tc_fence_after();
            const int gr = m0 + row;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + c * 32, r);
                const int gc = n0 + c * 32;
                if (gr < M && gc < N) {
                    if (out_dtype == SANIC_BF16) {
                        uint32_t pk[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            pk[j] = pack_bf16x2(__uint_as_float(r[2 * j]) * rstd, __uint_as_float(r[2 * j + 1]) * rstd);
                        uint16_t* dst = (uint16_t*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N && wide_ok) {
#pragma unroll
                            for (int j = 0; j < 2; ++j)      // 32-byte stores: every lane writes whole sectors
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16 * j), "r"(pk[8 * j]),
                                             "r"(pk[8 * j + 1]), "r"(pk[8 * j + 2]), "r"(pk[8 * j + 3]), "r"(pk[8 * j + 4]),
                                             "r"(pk[8 * j + 5]), "r"(pk[8 * j + 6]), "r"(pk[8 * j + 7]) : "memory");
                        } else if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *(uint4*)(dst + 8 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j)
                                dst[j] = (uint16_t)((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xFFFF));
                        }
                    } else {
                        float* dst = (float*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *(float4*)(dst + 4 * j) = make_float4(__uint_as_float(r[4 * j]) * rstd, __uint_as_float(r[4 * j + 1]) * rstd,
                                                                      __uint_as_float(r[4 * j + 2]) * rstd, __uint_as_float(r[4 * j + 3]) * rstd);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j) dst[j] = __uint_as_float(r[j]) * rstd;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&sh->tmem_empty); mbar_arrive(&sh->ss_empty[a]); }
        }
    }
    // teardown: every role has left its loop (normally or after a bounded wait ran out)
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

// ───────────────────────── the same contraction on a pair of SMs ─────────────────────────
// Two CTAs of a cluster share one 256x256 output tile: CTA r holds rows [128r, 128r+128) of A and columns
// [128r, 128r+128) of B in its shared memory, and ONE thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256):
// each SM multiplies its half of A with the whole of B, reading the other half of B from its peer. Per k-block a CTA
// brings 32 KB through L2 -> shared memory instead of 48 KB for the same tensor work, which is what bounds the one-CTA
// tile. With B's shared-memory traffic halved there is room to rewrite A in place (x*g back to the same swizzled
// bytes) and feed the MMA from shared memory; tensor memory then holds TWO 256-column accumulators and the epilogue
// of a tile overlaps the main loop of the next. (Fed from tensor memory instead, the MMAs paid a fixed cost per
// instruction and left room for one accumulator only: same speed, epilogue exposed.)
// Six stages of (A 16 KB + B half 16 KB); A and B have their own producer threads and full barriers, one empty barrier.
// Two groups of 8 transform warps take alternate k-blocks. bf16 output leaves through shared-memory staging and one
// bulk tensor store per 32 x 32 block.
// Synchronisation across the pair: the transform warps of both CTAs arrive on the LEADER's ready barrier with relaxed
// cluster-scope arrivals (a release fence on that path costs about 0.9 us per arrival); the leader commits each stage
// to its own empty barrier and a relay thread forwards it to the peer's; the accumulator-full commits go to both CTAs
// (one commit per destination); the epilogue warps of both CTAs arrive on the leader's accumulator-empty barrier.
constexpr int PA_SLOTS = 6;                            // A tiles in shared memory, transformed in place, read by the MMA from there
constexpr int PB_SLOTS = 6;                            // B half-tiles in shared memory; stage s = A slot s + B slot s
constexpr int PB_BYTES = (BN / 2) * BK * 2;            // 16 KB: this CTA's half of the B tile
constexpr int P_RING_BYTES = PA_SLOTS * A_BYTES + PB_SLOTS * PB_BYTES;    // 192 KB
constexpr int P_OUT_BYTES = 8 * 2048;                  // store staging: one 32 x 32 bf16 block per epilogue warp
constexpr int P_NTHREADS = 896;                        // warps 0-3 single-thread roles, 4-19 A transform (two groups), 20-27 epilogue

struct PShared {
    uint64_t full_a[PA_SLOTS];
    uint64_t full_b[PB_SLOTS], ready[PB_SLOTS], empty[PB_SLOTS];
    uint64_t tmem_full[2], tmem_empty[2], ss_full[2], ss_empty[2];
    uint32_t tmem_base;
    volatile int abort_flag;
    float ss[2][4][BM];   // [accumulator use parity][transform group * 2 + row half][row]
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same without the release fence, for a thread that only passes on an event it has itself acquired (the facts it
// forwards are completed tensor-core reads or tcgen05.st / TMA writes that their issuers already waited for).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bounded wait. CLUSTER: acquire at cluster scope, for barriers whose arrivals may come from the peer CTA (it costs more
// than the CTA-scope form, so only the roles that need it use it).
template <bool CLUSTER>
__device__ __forceinline__ bool mbar_wait_p(uint64_t* bar, uint32_t parity, PShared* sh, int* err, int code) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < P_SPIN_LIMIT; ++it) {
        uint32_t done;
        if (CLUSTER)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u && sh->abort_flag) return false;
    }
    sh->abort_flag = 1;
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on ONE barrier, given by its shared::cluster address (this CTA's or the peer's), when the pair's MMAs so far retire
__device__ __forceinline__ void umma2_commit(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

__global__ void __launch_bounds__(P_NTHREADS, 1)
gemm_rmsnorm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_y, const uint16_t* __restrict__ gamma, void* __restrict__ y,
                         int M, int N, int K, int w_is_nk, float eps, int out_dtype, int* err, int gamma_bytes, int bulk_store,
                         int prescaled) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* aligned = smem_dyn + (base - raw);
    uint16_t* gsm = (uint16_t*)(aligned + P_RING_BYTES);
    const uint32_t b_ring = base + PA_SLOTS * A_BYTES;
    // after gamma: 8 x 2 KB of store staging (one 32 x 32 bf16 block per epilogue warp) when bulk_store, then the barriers
    const uint32_t stage_out = base + P_RING_BYTES + gamma_bytes;
    PShared* sh = (PShared*)(aligned + P_RING_BYTES + gamma_bytes + (bulk_store ? P_OUT_BYTES : 0));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                  // 0 = the leader, which issues every MMA
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int kblocks = (K + BK - 1) / BK;
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PA_SLOTS; ++s) mbar_init(&sh->full_a[s], 1);
        for (int s = 0; s < PB_SLOTS; ++s) { mbar_init(&sh->full_b[s], 1); mbar_init(&sh->ready[s], 16); mbar_init(&sh->empty[s], prescaled ? 9 : 1); }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 16);
            mbar_init(&sh->ss_full[a], 16); mbar_init(&sh->ss_empty[a], 8);
        }
        sh->abort_flag = 0;
        sh->tmem_base = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (!prescaled)
        for (int i = threadIdx.x; i < kblocks * BK; i += P_NTHREADS) gsm[i] = (i < K) ? gamma[i] : (uint16_t)0;
    __syncthreads();
    if (warp == 3) {
        // one warp of EACH CTA of the pair allocates (all 512 columns, so both get base 0)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ── TMA producer for A: this CTA's 128 rows; a slot is free again once the pair's MMAs on it retire ──
        if (lane == 0) {
            int stage = 0; uint32_t phase = 1;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs) {
                const int m0 = (t % m_tiles) * (2 * BM) + (int)rank * BM;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait_p<true>(&sh->empty[stage], phase, sh, err, 20);
                    if (!ok) break;
                    mbar_expect_tx(&sh->full_a[stage], A_BYTES);
                    tma_load_2d(base + stage * A_BYTES, &map_a, &sh->full_a[stage], kb * BK, m0);
                    if (++stage == PA_SLOTS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 2) {
        // ── TMA producer for B: this CTA's 128 columns; a slot is free again once the pair's MMAs on it retire ──
        if (lane == 0) {
            int stage = 0; uint32_t phase = 1;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs) {
                const int n0 = (t / m_tiles) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait_p<true>(&sh->empty[stage], phase, sh, err, 21);
                    if (!ok) break;
                    const uint32_t sb = b_ring + stage * PB_BYTES;
                    mbar_expect_tx(&sh->full_b[stage], PB_BYTES);
                    if (w_is_nk) {
                        tma_load_2d(sb, &map_b, &sh->full_b[stage], kb * BK, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d(sb + j * (64 * BK * 2), &map_b, &sh->full_b[stage], n0 + 64 * j, kb * BK);
                    }
                    if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ── MMA issuer: the leader CTA only ──
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((w_is_nk ? 0u : 1u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            int stage = 0; uint32_t phase = 0;
            int use = 0;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs, ++use) {
                const int ab = use & 1;                                                   // accumulator buffer: 256 columns each
                ok = mbar_wait_p<true>(&sh->tmem_empty[ab], ((use >> 1) & 1) ^ 1, sh, err, 22);    // both epilogues have read its previous tile
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)ab * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait_p<true>(&sh->ready[stage], phase, sh, err, 23);      // both CTAs' A halves are in tensor memory, both B halves landed
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sb = b_ring + stage * PB_BYTES;
                    const uint64_t adesc = make_desc(base + stage * A_BYTES, 16, 1024);
                    const uint64_t bdesc = w_is_nk ? make_desc(sb, 16, 1024) : make_desc(sb, 64 * BK * 2, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t bd = bdesc + (uint64_t)(w_is_nk ? k * 2 : k * 128);
                        umma2_f16_ss(acc, adesc + (uint64_t)(k * 2), bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    // one commit per stage, to the leader's own barrier; warp 3 relays it to the peer
                    umma2_commit(map_to_rank(smem_u32(&sh->empty[stage]), 0));
                    if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
                }
                if (ok) {
                    const uint32_t f = smem_u32(&sh->tmem_full[ab]);
                    umma2_commit(map_to_rank(f, 0));
                    umma2_commit(map_to_rank(f, 1));
                }
            }
        }
    } else if (warp == 3) {
        // ── leader only: relay "stage free" to the peer's producer (a second commit per stage would cost the issuer more) ──
        if (lane == 0 && rank == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; t < tiles && ok; t += n_pairs) {
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait_p<true>(&sh->empty[stage], phase, sh, err, 29);
                    if (!ok) break;
                    mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&sh->empty[stage]), 1));
                    if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp >= 4 && warp < 20) {
        // ── A transform (both CTAs): shared memory -> x*g -> this CTA's tensor memory, sum x^2 ──
        // Two groups of 8 warps take alternate k-blocks: one k-block costs a warp about 1000 clocks of mostly latency
        // (barrier wake-ups, shared-memory loads, the tensor-memory store and its wait), twice what the tensor core needs.
        const int idx = (threadIdx.x - 128) & 255, group = (threadIdx.x - 128) >> 8;
        const int row = idx & (BM - 1), half = idx >> 7;
        int use = 0;
        uint32_t gk = 0;                     // k-blocks since the start, over all tiles: ring positions derive from it
        bool ok = true;
        for (int t = pair; t < tiles && ok; t += n_pairs, ++use) {
            const int a = use & 1;
            float ss = 0.0f;
            for (int kb = 0; kb < kblocks; ++kb, ++gk) {
                if ((int)(gk & 1u) != group) continue;
                const int stage = gk % PB_SLOTS; const uint32_t phase = (gk / PB_SLOTS) & 1u;
                ok = mbar_wait_p<false>(&sh->full_a[stage], phase, sh, err, 24);
                if (!ok) break;
                unsigned char* arow = aligned + stage * A_BYTES + row * 128;
                if (prescaled) {
                    // The weights already carry g: the MMA reads x as the TMA left it, so the stage is vouched for BEFORE
                    // this warp reads it (the transform leaves the ring's latency cycle); what remains here is sum x^2,
                    // and the stage's empty barrier also counts these 8 warps so the producer cannot overtake the read.
                    ok = mbar_wait_p<false>(&sh->full_b[stage], phase, sh, err, 31);
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&sh->ready[stage]), 0));
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const int c = half * 4 + c4;
                        const uint4 v = *(const uint4*)(arow + ((c ^ (row & 7)) << 4));
                        const uint32_t xs[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float x0 = bf16lo(xs[j]), x1 = bf16hi(xs[j]);
                            ss = fmaf(x0, x0, ss); ss = fmaf(x1, x1, ss);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->empty[stage]);
                    continue;
                }
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const int c = half * 4 + c4;
                    const uint4 v = *(const uint4*)(arow + ((c ^ (row & 7)) << 4));
                    const uint4 gv = *(const uint4*)(gsm + kb * BK + c * 8);
                    uint32_t xs[4] = {v.x, v.y, v.z, v.w};
                    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float x0 = bf16lo(xs[j]), x1 = bf16hi(xs[j]);
                        ss = fmaf(x0, x0, ss); ss = fmaf(x1, x1, ss);
                        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(xs[j]) : "r"(xs[j]), "r"(gs[j]));
                    }
                    // back to the same (swizzled) place: the MMA reads x*g from shared memory
                    *(uint4*)(arow + ((c ^ (row & 7)) << 4)) = make_uint4(xs[0], xs[1], xs[2], xs[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> visible to the tensor core's reads
                // the arrival below also vouches for this CTA's half of B
                ok = mbar_wait_p<false>(&sh->full_b[stage], phase, sh, err, 31);
                if (!ok) break;
                __syncwarp();
                // The peer's warps arrive on the leader's barrier directly, without a release fence (it cost about 0.9 us per
                // arrival): the writes above were ordered by the proxy fence, the TMA bytes were observed through full_b
                if (lane == 0) mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&sh->ready[stage]), 0));
            }
            if (!ok) break;
            ok = mbar_wait_p<false>(&sh->ss_empty[a], ((use >> 1) & 1) ^ 1, sh, err, 25);
            if (!ok) break;
            sh->ss[a][group * 2 + half][row] = ss;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->ss_full[a]);
        }
    } else if (warp >= 20) {
        // ── epilogue (both CTAs): this CTA's 128 rows of the 256 x 256 tile; two warps per lane quarter, 128 columns each ──
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int c_begin = ((warp - 20) >> 2) * (BN / 64);
        const bool wide_ok = (N % 16 == 0) && (((uintptr_t)y & 31) == 0);     // 32-byte stores need 32-byte aligned rows
        int use = 0;
        bool ok = true;
        const float inv_k = 1.0f / (float)K;
        for (int t = pair; t < tiles && ok; t += n_pairs, ++use) {
            const int a = use & 1;
            const int m0 = (t % m_tiles) * (2 * BM) + (int)rank * BM, n0 = (t / m_tiles) * BN;
            ok = mbar_wait_p<false>(&sh->ss_full[a], (use >> 1) & 1, sh, err, 26);
            if (!ok) break;
            const float ssv = (sh->ss[a][0][row] + sh->ss[a][1][row]) + (sh->ss[a][2][row] + sh->ss[a][3][row]);
            const float rstd = 1.0f / sqrtf(ssv * inv_k + eps);
            ok = mbar_wait_p<false>(&sh->tmem_full[a], (use >> 1) & 1, sh, err, 27);     // parked, not polling: 256 threads wait here for a whole tile
            if (!ok) break;
            tc_fence_after();
            const int gr = m0 + row;
#pragma unroll 1
            for (int c = c_begin; c < c_begin + BN / 64; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)a * BN + c * 32, r);
                const int gc = n0 + c * 32;
                if (bulk_store) {
                    // bf16 through shared memory and one bulk tensor store per 32 x 32 block: the warp hands 2 KB to the copy
                    // engine instead of issuing 32-row scattered stores (which cost 4 us of a 20 us tile); the engine clips
                    // the block at the edges of y
                    const uint32_t mine = stage_out + (uint32_t)(warp - 20) * 2048u;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // the previous block has been read out
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t p0 = pack_bf16x2(__uint_as_float(r[8 * j]) * rstd, __uint_as_float(r[8 * j + 1]) * rstd);
                        const uint32_t p1 = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * rstd, __uint_as_float(r[8 * j + 3]) * rstd);
                        const uint32_t p2 = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * rstd, __uint_as_float(r[8 * j + 5]) * rstd);
                        const uint32_t p3 = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * rstd, __uint_as_float(r[8 * j + 7]) * rstd);
                        // 64-byte rows: the 16-byte chunk index is XORed with (row / 2) % 4, the copy engine's 64-byte swizzle
                        const uint32_t at = mine + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && gc < N && m0 + q * 32 < M) {
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                     ::"l"((uint64_t)&map_y), "r"(gc), "r"(m0 + q * 32), "r"(mine) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (gr < M && gc < N) {
                    if (out_dtype == SANIC_BF16) {
                        uint32_t pk[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            pk[j] = pack_bf16x2(__uint_as_float(r[2 * j]) * rstd, __uint_as_float(r[2 * j + 1]) * rstd);
                        uint16_t* dst = (uint16_t*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N && wide_ok) {
#pragma unroll
                            for (int j = 0; j < 2; ++j)      // 32-byte stores: every lane writes whole sectors
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16 * j), "r"(pk[8 * j]),
                                             "r"(pk[8 * j + 1]), "r"(pk[8 * j + 2]), "r"(pk[8 * j + 3]), "r"(pk[8 * j + 4]),
                                             "r"(pk[8 * j + 5]), "r"(pk[8 * j + 6]), "r"(pk[8 * j + 7]) : "memory");
                        } else if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *(uint4*)(dst + 8 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j)
                                dst[j] = (uint16_t)((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xFFFF));
                        }
                    } else {
                        float* dst = (float*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *(float4*)(dst + 4 * j) = make_float4(__uint_as_float(r[4 * j]) * rstd, __uint_as_float(r[4 * j + 1]) * rstd,
                                                                      __uint_as_float(r[4 * j + 2]) * rstd, __uint_as_float(r[4 * j + 3]) * rstd);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j) dst[j] = __uint_as_float(r[j]) * rstd;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&sh->tmem_empty[a]), 0)); mbar_arrive(&sh->ss_empty[a]); }
        }
    }
    if (bulk_store && warp >= 20 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every block of y has been written
    // teardown: neither CTA may leave (or free tensor memory) while the other can still reach into it
    tc_fence_before();
    cluster_sync_all();
    if (warp == 3) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

// ───────────────────────── the pair tile with A brought in through registers ─────────────────────────
// Same 256x256 tile on a pair of SMs, same accumulators and epilogue; selected with SANIC_GEMM_PAIR=2. It moves fewer
// bytes through shared memory than the kernel above (per k-block and SM: 16 KB of A stored once from registers instead of
// copied in, read, multiplied and written back) and measures the same (131 against 128 us at 4096 x 2048 x 8192), which
// is why the kernel above stays the default: at this tile neither form is bound by bytes but by chains of shared-memory
// and barrier latencies that the tensor core's own operand reads stretch (measured in this kernel with clock counters, on
// the thread concerned, while the MMAs run: a satisfied mbarrier wait 210 clocks, a shared-memory load 55, a tcgen05.mma
// issue 60-130, sixteen bytes stored per lane 30, dependent ALU instructions of a transform warp 4.5 each).
//   * A never waits in shared memory for data: four groups of transform warps take every fourth k-block; a warp loads x
//     from global memory into REGISTERS one of its k-blocks ahead, multiplies by g and takes sum x^2 while the slot may
//     still be busy, and stores the swizzled tile when the slot frees (a slot's life starts at the store);
//   * both CTAs' B copies complete on the LEADER's barrier (cp.async.bulk.tensor.cta_group::2 with the leader's mbarrier),
//     so no warp has to vouch for B;
//   * one tcgen05.commit per stage frees the slot in both CTAs (mbarrier multicast of the commit), no relay;
//   * the MMA thread waits on no barrier inside a tile: watcher threads turn barrier completions into counters (the
//     peer's through one posted store into the leader's shared memory per k-block), and one read of the counters often
//     covers several k-blocks.
// With gamma == NULL (weights scaled beforehand) the same path runs without the multiply.
constexpr int P2_GROUPS = 4;          // groups of transform warps; each takes every P2_GROUPS-th k-block
struct P2Shared {
    uint64_t full_b[PB_SLOTS], ready[PB_SLOTS], empty[PB_SLOTS];
    uint64_t tmem_full[2], tmem_empty[2], ss_full[2], ss_empty[2];
    uint32_t tmem_base;
    volatile int abort_flag;
    // k-blocks (of the pair's sequence) whose B halves have landed / whose A half is stored in this CTA / in the peer
    // (the leader's copies are the ones read; the peer writes seen_a_peer into the leader's shared memory)
    uint32_t seen_b, seen_a, seen_a_peer;
    float ss[2][P2_GROUPS][BM];   // [accumulator use parity][transform group][row]
};
template <bool CLUSTER>
__device__ __forceinline__ bool mbar_wait_p2(uint64_t* bar, uint32_t parity, P2Shared* sh, int* err, int code) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < P_SPIN_LIMIT; ++it) {
        uint32_t done;
        if (CLUSTER)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        else
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u && sh->abort_flag) return false;
    }
    sh->abort_flag = 1;
    atomicCAS(err, 0, code);
    return false;
}
// one lane waits for the warp: 31 fewer pollers on the barrier per warp
template <bool CLUSTER>
__device__ __forceinline__ bool warp_wait_p2(uint64_t* bar, uint32_t parity, P2Shared* sh, int* err, int code, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait_p2<CLUSTER>(bar, parity, sh, err, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// this CTA's copy, completion counted on the mbarrier at `bar_cluster_addr` (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
// arrives on the barrier at this offset in BOTH CTAs of the pair when the pair's MMAs so far retire
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// PROF: the roles of pair 0 count clocks in registers and write them to `prof` when they leave (what the profile entry
// point reports): [0] k-blocks issued, [1] the MMA thread's clocks over its whole loop, [2] of those, clocks reading the
// progress counters, [3] counter reads, [4] clocks waiting for a free accumulator; [5] the B producer's clocks waiting for a
// free slot; for transform warp 0 of the leader [6..11] and of the peer [12..17]: its k-blocks, clocks in arithmetic (with
// the wait for its loads), waiting for the slot, storing, in the proxy fence, in the arrival.
template <bool PROF>
__global__ void __launch_bounds__(P_NTHREADS, 1)
gemm_rmsnorm_pair_reg_kernel(const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_y,
                             const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma, void* __restrict__ y,
                             int M, int N, int K, int w_is_nk, float eps, int out_dtype, int* err, int gamma_bytes, int bulk_store,
                             unsigned long long* prof) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* aligned = smem_dyn + (base - raw);
    uint16_t* gsm = (uint16_t*)(aligned + P_RING_BYTES);
    const uint32_t b_ring = base + PA_SLOTS * A_BYTES;
    const uint32_t stage_out = base + P_RING_BYTES + gamma_bytes;
    P2Shared* sh = (P2Shared*)(aligned + P_RING_BYTES + gamma_bytes + (bulk_store ? P_OUT_BYTES : 0));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int kblocks = (K + BK - 1) / BK;
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const bool scaled = gamma != nullptr;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PB_SLOTS; ++s) { mbar_init(&sh->full_b[s], 1); mbar_init(&sh->ready[s], 16 / P2_GROUPS); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh->tmem_full[a], 1); mbar_init(&sh->tmem_empty[a], 16);
            mbar_init(&sh->ss_full[a], 16); mbar_init(&sh->ss_empty[a], 8);
        }
        sh->abort_flag = 0;
        sh->tmem_base = 0;
        sh->seen_a = 0; sh->seen_b = 0; sh->seen_a_peer = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (scaled)
        for (int i = threadIdx.x; i < kblocks * BK; i += P_NTHREADS) gsm[i] = (i < K) ? gamma[i] : (uint16_t)0;
    __syncthreads();
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp == 0) {
        // ── TMA producer for B: this CTA's 128 columns into its own shared memory, bytes counted on the leader's barrier ──
        if (lane == 0) {
            int stage = 0; uint32_t phase = 1;
            bool ok = true;
            long long t_wait = 0;
            for (int t = pair; t < tiles && ok; t += n_pairs) {
                const int n0 = (t / m_tiles) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < kblocks; ++kb) {
                    const long long c0 = PROF ? clock64() : 0;
                    ok = mbar_wait_p2<false>(&sh->empty[stage], phase, sh, err, 21);
                    if (PROF) t_wait += clock64() - c0;
                    if (!ok) break;
                    const uint32_t sb = b_ring + stage * PB_BYTES;
                    const uint32_t bar = map_to_rank(smem_u32(&sh->full_b[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&sh->full_b[stage], 2 * PB_BYTES);      // both halves
                    if (w_is_nk) {
                        tma_load_2d_pair(sb, &map_b, bar, kb * BK, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j)
                            tma_load_2d_pair(sb + j * (64 * BK * 2), &map_b, bar, n0 + 64 * j, kb * BK);
                    }
                    if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
                }
            }
            if (PROF && blockIdx.x == 0) prof[5] = (unsigned long long)t_wait;
        }
    } else if (warp == 1) {
        // ── MMA issuer: the leader CTA only ──
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((w_is_nk ? 0u : 1u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            int stage = 0; uint32_t phase = 0;
            int use = 0;
            bool ok = true;
            uint32_t q = 0, avail = 0;
            long long t_read = 0, n_read = 0, t_acc = 0;
            const long long t_begin = PROF ? clock64() : 0;
            for (int t = pair; t < tiles && ok; t += n_pairs, ++use) {
                const int ab = use & 1;
                const long long c9 = PROF ? clock64() : 0;
                ok = mbar_wait_p2<true>(&sh->tmem_empty[ab], ((use >> 1) & 1) ^ 1, sh, err, 22);
                if (PROF) t_acc += clock64() - c9;
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)ab * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (q >= avail) {
                        // one plain shared-memory read per counter instead of two mbarrier waits (a satisfied mbarrier wait costs
                        // this thread about 210 clocks, a shared-memory load 55): the watcher threads below turn barrier
                        // completions into counters, and one read often covers several k-blocks
                        uint32_t it = 0;
                        const long long c0 = PROF ? clock64() : 0;
                        for (;;) {
                            uint32_t pa, pp, pb;
                            asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(pa) : "r"(smem_u32(&sh->seen_a)) : "memory");
                            asm volatile("ld.acquire.cluster.shared.u32 %0, [%1];" : "=r"(pp) : "r"(smem_u32(&sh->seen_a_peer)) : "memory");
                            asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(pb) : "r"(smem_u32(&sh->seen_b)) : "memory");
                            avail = pa < pb ? pa : pb;
                            avail = avail < pp ? avail : pp;
                            if (q < avail) break;
                            if (++it > P_SPIN_LIMIT || ((it & 1023u) == 0 && sh->abort_flag)) { if (it > P_SPIN_LIMIT) { sh->abort_flag = 1; atomicCAS(err, 0, 23); } ok = false; break; }
                        }
                        if (!ok) break;
                        if (PROF) { t_read += clock64() - c0; ++n_read; }
                    }
                    const uint32_t sb = b_ring + stage * PB_BYTES;
                    const uint64_t adesc = make_desc(base + stage * A_BYTES, 16, 1024);
                    const uint64_t bdesc = w_is_nk ? make_desc(sb, 16, 1024) : make_desc(sb, 64 * BK * 2, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t bd = bdesc + (uint64_t)(w_is_nk ? k * 2 : k * 128);
                        umma2_f16_ss(acc, adesc + (uint64_t)(k * 2), bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma2_commit_both(&sh->empty[stage]);
                    ++q;
                    if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
                }
                if (ok) umma2_commit_both(&sh->tmem_full[ab]);
            }
            if (PROF && blockIdx.x == 0) {
                prof[0] = q; prof[1] = (unsigned long long)(clock64() - t_begin); prof[2] = (unsigned long long)t_read;
                prof[3] = (unsigned long long)n_read; prof[4] = (unsigned long long)t_acc;
            }
        }
    } else if (warp == 2 || warp == 3) {
        // ── watchers: turn barrier completions into counters in the LEADER's shared memory. Leader warp 2: B landed (both
        // halves, counted by the copies themselves); warp 3 of each CTA: this CTA's A half stored (the peer writes its
        // counter across the cluster: one posted store per k-block instead of a remote barrier arrival per warp, which
        // held each arriving warp for about 800 clocks) ──
        if (lane == 0 && (rank == 0 || warp == 3)) {
            uint64_t* bars = warp == 2 ? sh->full_b : sh->ready;
            const uint32_t out = map_to_rank(smem_u32(warp == 2 ? &sh->seen_b : (rank == 0 ? &sh->seen_a : &sh->seen_a_peer)), 0);
            int stage = 0; uint32_t phase = 0;
            const int my_tiles = pair < tiles ? (tiles - pair + n_pairs - 1) / n_pairs : 0;
            const uint32_t total = (uint32_t)(my_tiles * kblocks);
            for (uint32_t q = 0; q < total; ++q) {
                if (!mbar_wait_p2<false>(&bars[stage], phase, sh, err, warp == 2 ? 28 : 29)) break;
                if (rank == 0) asm volatile("st.release.cta.shared::cluster.u32 [%0], %1;" ::"r"(out), "r"(q + 1) : "memory");
                else asm volatile("st.relaxed.cluster.shared::cluster.u32 [%0], %1;" ::"r"(out), "r"(q + 1) : "memory");
                if (++stage == PB_SLOTS) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp >= 4 && warp < 20) {
        // ── A (both CTAs): global memory -> registers -> x*g -> swizzled shared memory, sum x^2 ──
        // P2_GROUPS groups of warps take every P2_GROUPS-th k-block of the pair's sequence (over all its tiles): a k-block costs
        // a warp a chain of latencies (barrier wake-up, the loads' arrival, stores, the proxy fence, the arrival at the
        // leader) of about 900 clocks, and the tensor cores want one every 512. A warp covers rows 4w..4w+3 of each 16-row
        // band: 8 lanes per row, 16 bytes each, so a load instruction reads four whole 128-byte rows.
        constexpr int WPG = 16 / P2_GROUPS, RPT = 32 / WPG;          // warps per group; rows per thread
        const int group = (warp - 4) / WPG, wg = (warp - 4) % WPG;
        const int c = lane & 7;                        // 16-byte chunk of the row
        const int r0 = wg * 4 + (lane >> 3);           // row within a (4 * WPG)-row band; rows r0 + 4 * WPG * j
        const uint32_t swz = (uint32_t)((c ^ (r0 & 7)) << 4);
        const int my_tiles = pair < tiles ? (tiles - pair + n_pairs - 1) / n_pairs : 0;
        float ss[RPT];
#pragma unroll
        for (int j = 0; j < RPT; ++j) ss[j] = 0.0f;
        bool ok = true;
        // the load stream runs one of this group's k-blocks ahead of the store stream; both walk (tile use, k-block) by P2_GROUPS
        int f_use = 0, f_kb = group, s_use = 0, s_kb = group, stage = group % PA_SLOTS;
        uint32_t phase = 1;                            // producer parity: the first pass over the ring does not wait
        while (f_kb >= kblocks && f_use < my_tiles) { f_kb -= kblocks; ++f_use; }
        while (s_kb >= kblocks && s_use < my_tiles) { s_kb -= kblocks; ++s_use; }
        auto row_base = [&](int use) { const int t = pair + use * n_pairs; return (t % m_tiles) * (2 * BM) + (int)rank * BM + r0; };
        int f_row = f_use < my_tiles ? row_base(f_use) : 0;
        uint4 buf[RPT];
        auto fetch = [&]() {
            if (f_use >= my_tiles) return;
            const int k0 = f_kb * BK + c * 8;
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                const int gr = f_row + 4 * WPG * j;
                buf[j] = (gr < M && k0 < K) ? __ldg((const uint4*)(x + (size_t)gr * K + k0)) : make_uint4(0, 0, 0, 0);
            }
            f_kb += P2_GROUPS;
            if (f_kb >= kblocks) {
                do { f_kb -= kblocks; ++f_use; } while (f_kb >= kblocks);
                if (f_use < my_tiles) f_row = row_base(f_use);
            }
        };
        auto flush = [&](int use) -> bool {            // this group's sum x^2 of tile `use` to the epilogue
            const int a = use & 1;
            if (!warp_wait_p2<false>(&sh->ss_empty[a], ((use >> 1) & 1) ^ 1, sh, err, 25, lane)) return false;
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                float v = ss[j];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (c == 0) sh->ss[a][group][r0 + 4 * WPG * j] = v;
                ss[j] = 0.0f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->ss_full[a]);
            return true;
        };
        int flushed = 0;
        long long t_math = 0, t_slot = 0, t_store = 0, t_fence = 0, t_arrive = 0, n_own = 0;
        fetch();
        while (s_use < my_tiles && ok) {
            while (flushed < s_use && ok) { ok = flush(flushed); ++flushed; }
            if (!ok) break;
            const long long c0 = PROF ? clock64() : 0;
            // multiply and square while the slot may still be busy: only the stores wait for it
            uint4 gv = make_uint4(0, 0, 0, 0);
            if (scaled) gv = *(const uint4*)(gsm + s_kb * BK + c * 8);
            const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int j = 0; j < RPT; ++j) {
                uint32_t xs[4] = {buf[j].x, buf[j].y, buf[j].z, buf[j].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x0 = bf16lo(xs[e]), x1 = bf16hi(xs[e]);
                    ss[j] = fmaf(x0, x0, ss[j]); ss[j] = fmaf(x1, x1, ss[j]);
                    // bf16 x bf16 is exact in f32, so the packed multiply equals bf16(float(x) * float(g)) bit for bit
                    if (scaled) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(xs[e]) : "r"(xs[e]), "r"(gs[e]));
                }
                buf[j] = make_uint4(xs[0], xs[1], xs[2], xs[3]);
            }
            const long long c1 = PROF ? clock64() : 0;
            ok = warp_wait_p2<false>(&sh->empty[stage], phase, sh, err, 24, lane);      // the pair's MMAs on this slot retired
            if (!ok) break;
            const long long c2 = PROF ? clock64() : 0;
            const uint32_t slot = base + stage * A_BYTES + (uint32_t)r0 * 128u + swz;
#pragma unroll
            for (int j = 0; j < RPT; ++j)
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(slot + (uint32_t)(4 * WPG * j) * 128u),
                             "r"(buf[j].x), "r"(buf[j].y), "r"(buf[j].z), "r"(buf[j].w) : "memory");
            const long long c3 = PROF ? clock64() : 0;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> visible to the tensor core's reads
            const long long c4 = PROF ? clock64() : 0;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->ready[stage]);       // this CTA's barrier; its watcher tells the leader
            if (PROF) {
                const long long c5 = clock64();
                t_math += c1 - c0; t_slot += c2 - c1; t_store += c3 - c2; t_fence += c4 - c3; t_arrive += c5 - c4; ++n_own;
            }
            fetch();                                   // the next of this group's k-blocks, in flight until its slot frees
            s_kb += P2_GROUPS;
            while (s_kb >= kblocks) { s_kb -= kblocks; ++s_use; }
            stage += P2_GROUPS;
            if (stage >= PA_SLOTS) { stage -= PA_SLOTS; phase ^= 1; }
        }
        while (ok && flushed < my_tiles) { ok = flush(flushed); ++flushed; }
        if (PROF && blockIdx.x < 2 && warp == 4 && lane == 0) {
            unsigned long long* o = prof + 6 + 6 * blockIdx.x;
            o[0] = (unsigned long long)n_own; o[1] = (unsigned long long)t_math; o[2] = (unsigned long long)t_slot;
            o[3] = (unsigned long long)t_store; o[4] = (unsigned long long)t_fence; o[5] = (unsigned long long)t_arrive;
        }
    } else if (warp >= 20) {
        // ── epilogue (both CTAs): this CTA's 128 rows of the 256 x 256 tile; two warps per lane quarter, 128 columns each ──
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int c_begin = ((warp - 20) >> 2) * (BN / 64);
        const bool wide_ok = (N % 16 == 0) && (((uintptr_t)y & 31) == 0);
        int use = 0;
        bool ok = true;
        const float inv_k = 1.0f / (float)K;
        for (int t = pair; t < tiles && ok; t += n_pairs, ++use) {
            const int a = use & 1;
            const int m0 = (t % m_tiles) * (2 * BM) + (int)rank * BM, n0 = (t / m_tiles) * BN;
            ok = mbar_wait_p2<false>(&sh->ss_full[a], (use >> 1) & 1, sh, err, 26);
            if (!ok) break;
            float ssv = 0.0f;
#pragma unroll
            for (int gI = 0; gI < P2_GROUPS; ++gI) ssv += sh->ss[a][gI][row];
            const float rstd = 1.0f / sqrtf(ssv * inv_k + eps);
            ok = mbar_wait_p2<false>(&sh->tmem_full[a], (use >> 1) & 1, sh, err, 27);
            if (!ok) break;
            tc_fence_after();
            const int gr = m0 + row;
#pragma unroll 1
            for (int cc = c_begin; cc < c_begin + BN / 64; ++cc) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)a * BN + cc * 32, r);
                const int gc = n0 + cc * 32;
                if (bulk_store) {
                    // bf16 through shared memory and one bulk tensor store per 32 x 32 block; the copy engine clips the
                    // block at the edges of y
                    const uint32_t mine = stage_out + (uint32_t)(warp - 20) * 2048u;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // the previous block has been read out
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t p0 = pack_bf16x2(__uint_as_float(r[8 * j]) * rstd, __uint_as_float(r[8 * j + 1]) * rstd);
                        const uint32_t p1 = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * rstd, __uint_as_float(r[8 * j + 3]) * rstd);
                        const uint32_t p2 = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * rstd, __uint_as_float(r[8 * j + 5]) * rstd);
                        const uint32_t p3 = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * rstd, __uint_as_float(r[8 * j + 7]) * rstd);
                        // 64-byte rows: the 16-byte chunk index is XORed with (row / 2) % 4, the copy engine's 64-byte swizzle
                        const uint32_t at = mine + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(p0), "r"(p1), "r"(p2), "r"(p3) : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && gc < N && m0 + q * 32 < M) {
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                                     ::"l"((uint64_t)&map_y), "r"(gc), "r"(m0 + q * 32), "r"(mine) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (gr < M && gc < N) {
                    if (out_dtype == SANIC_BF16) {
                        uint32_t pk[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            pk[j] = pack_bf16x2(__uint_as_float(r[2 * j]) * rstd, __uint_as_float(r[2 * j + 1]) * rstd);
                        uint16_t* dst = (uint16_t*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N && wide_ok) {
#pragma unroll
                            for (int j = 0; j < 2; ++j)
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + 16 * j), "r"(pk[8 * j]),
                                             "r"(pk[8 * j + 1]), "r"(pk[8 * j + 2]), "r"(pk[8 * j + 3]), "r"(pk[8 * j + 4]),
                                             "r"(pk[8 * j + 5]), "r"(pk[8 * j + 6]), "r"(pk[8 * j + 7]) : "memory");
                        } else if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                *(uint4*)(dst + 8 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j)
                                dst[j] = (uint16_t)((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xFFFF));
                        }
                    } else {
                        float* dst = (float*)y + (size_t)gr * N + gc;
                        if (gc + 32 <= N) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                *(float4*)(dst + 4 * j) = make_float4(__uint_as_float(r[4 * j]) * rstd, __uint_as_float(r[4 * j + 1]) * rstd,
                                                                      __uint_as_float(r[4 * j + 2]) * rstd, __uint_as_float(r[4 * j + 3]) * rstd);
                        } else {
                            for (int j = 0; j < 32 && gc + j < N; ++j) dst[j] = __uint_as_float(r[j]) * rstd;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&sh->tmem_empty[a]), 0)); mbar_arrive(&sh->ss_empty[a]); }
        }
    }
    if (bulk_store && warp >= 20 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    // teardown: neither CTA may leave (or free tensor memory) while the other can still reach into it
    tc_fence_before();
    cluster_sync_all();
    if (warp == 3) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int32_t encode_2d(sanic_ctx* ctx, CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                  uint32_t box_outer, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    if (!ctx->encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || !fn) return sanic_fail(ctx, SANIC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
        ctx->encode_tiled = fn;
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((encode_fn)ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                                                strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return sanic_fail(ctx, SANIC_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    return SANIC_OK;
}
}  // namespace

namespace {
// W'[n, k] = bf16(W[n, k] * g[k]) (bf16 x bf16 is exact in f32, one rounding): eight elements per thread.
__global__ void __launch_bounds__(256) prescale_kernel(const uint4* __restrict__ w, const uint16_t* __restrict__ gamma, uint4* __restrict__ out,
                                                       size_t n8, int K, int N, int w_is_nk) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = w[i];
        uint32_t xs[4] = {v.x, v.y, v.z, v.w};
        if (w_is_nk) {                       // [N, K]: eight consecutive k of one row
            const int k = (int)((i * 8) % (size_t)K);
            const uint4 g = *(const uint4*)(gamma + k);
            const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(xs[j]) : "r"(xs[j]), "r"(gs[j]));
        } else {                             // [K, N]: eight consecutive n of one k
            const int k = (int)((i * 8) / (size_t)N);
            const uint32_t g2 = (uint32_t)gamma[k] * 0x00010001u;
#pragma unroll
            for (int j = 0; j < 4; ++j) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(xs[j]) : "r"(xs[j]), "r"(g2));
        }
        out[i] = make_uint4(xs[0], xs[1], xs[2], xs[3]);
    }
}
}  // namespace

extern "C" int32_t sanic_gemm_prescale_weights(sanic_ctx* ctx, const void* gamma, const void* w, void* w_out, int32_t N, int32_t K,
                                               int32_t w_is_nk, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, gamma && w && w_out && N > 0 && K > 0, "gemm_prescale_weights: bad arguments");
    SANIC_REQUIRE(ctx, K % 8 == 0 && N % 8 == 0, "gemm_prescale_weights: K and N must be multiples of 8");
    SANIC_REQUIRE(ctx, ((uintptr_t)w % 16) == 0 && ((uintptr_t)w_out % 16) == 0 && ((uintptr_t)gamma % 16) == 0,
                  "gemm_prescale_weights: tensors must be 16-byte aligned");
    sanic_set_device(ctx);
    const size_t n8 = (size_t)N * K / 8;
    const int blocks = (int)((n8 + 255) / 256 < (size_t)(8 * ctx->sm_count) ? (n8 + 255) / 256 : (size_t)(8 * ctx->sm_count));
    prescale_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)w, (const uint16_t*)gamma, (uint4*)w_out, n8, K, N, w_is_nk);
    SANIC_LAUNCH_CHECK(ctx, "gemm_prescale_weights");
    return SANIC_OK;
}

extern "C" int32_t sanic_gemm_rmsnorm(sanic_ctx* ctx, const sanic_gemm_rmsnorm_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->x && p->w && p->y, "gemm_rmsnorm: null tensor");
    SANIC_REQUIRE(ctx, p->M > 0 && p->N > 0 && p->K > 0, "gemm_rmsnorm: empty extent");
    SANIC_REQUIRE(ctx, p->K % 8 == 0 && p->N % 8 == 0, "gemm_rmsnorm: K and N must be multiples of 8 (16-byte rows)");
    SANIC_REQUIRE(ctx, p->K <= MAX_K, "gemm_rmsnorm: K is limited to 8192");
    SANIC_REQUIRE(ctx, ((uintptr_t)p->x % 16) == 0 && ((uintptr_t)p->w % 16) == 0 && ((uintptr_t)p->y % 16) == 0,
                  "gemm_rmsnorm: tensors must be 16-byte aligned");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_BF16 || p->out_dtype == SANIC_F32, "gemm_rmsnorm: output must be bf16 or f32");
    sanic_set_device(ctx);
    CUtensorMap map_a, map_b;
    int32_t rc = encode_2d(ctx, &map_a, p->x, (uint64_t)p->K, (uint64_t)p->M, BK, BM);
    if (rc != SANIC_OK) return rc;
    if (p->w_is_nk) rc = encode_2d(ctx, &map_b, p->w, (uint64_t)p->K, (uint64_t)p->N, BK, BN);
    else rc = encode_2d(ctx, &map_b, p->w, (uint64_t)p->N, (uint64_t)p->K, 64, BK);
    if (rc != SANIC_OK) return rc;

    cudaStream_t st = (cudaStream_t)stream;
    // The 256 x 256 tile on SM pairs wins (5-7 % at 4096 x 2048 x 8192) once there are enough of those tiles to fill the
    // pairs; smaller problems keep the one-CTA 128 x 256 tile. SANIC_GEMM_PAIR=0/1 forces the choice (tests, A/B timing).
    const int pair_tiles = ((p->M + 2 * BM - 1) / (2 * BM)) * ((p->N + BN - 1) / BN);
    const char* force = getenv("SANIC_GEMM_PAIR");
    // gamma == NULL: the weights were pre-scaled with sanic_gemm_prescale_weights (only the pair kernel has that form)
    const bool prescaled = (p->gamma == nullptr);
    const bool use_pair = prescaled || ctx->gemm_prof || (force ? (force[0] == '1' || force[0] == '2') : (p->M >= 4 * BM && pair_tiles >= ctx->sm_count / 2));
    if (use_pair) {
        // the 256 x 256 tile on a pair of SMs: B's map has a 128-row box (this CTA's half)
        if (p->w_is_nk) {
            rc = encode_2d(ctx, &map_b, p->w, (uint64_t)p->K, (uint64_t)p->N, BK, BN / 2);
            if (rc != SANIC_OK) return rc;
        }
        const int kb = (p->K + BK - 1) / BK;
        const int gamma_bytes = ((kb * BK * 2 + 1023) / 1024) * 1024;
        int psmem = P_RING_BYTES + gamma_bytes + (int)sizeof(PShared) + 1024;
        // bf16 output goes through staging and bulk tensor stores when shared memory has room for it (K up to 7168)
        const int bulk_store = (p->out_dtype == SANIC_BF16 && psmem + P_OUT_BYTES <= ctx->max_smem) ? 1 : 0;
        CUtensorMap map_y = map_a;
        if (bulk_store) {
            psmem += P_OUT_BYTES;
            rc = encode_2d(ctx, &map_y, p->y, (uint64_t)p->N, (uint64_t)p->M, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
            if (rc != SANIC_OK) return rc;
        }
        const bool reg_path = ctx->gemm_prof || (force && force[0] == '2');
        if (reg_path) {
            SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_rmsnorm_pair_reg_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem));
            SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_rmsnorm_pair_reg_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem));
        }
        SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_rmsnorm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem));
        const int ptiles = ((p->M + 2 * BM - 1) / (2 * BM)) * ((p->N + BN - 1) / BN);
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.blockDim = dim3(P_NTHREADS); cfg.dynamicSmemBytes = psmem; cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
        cfg.gridDim = dim3(2 * (ctx->sm_count / 2));
        int max_clusters = 0;
        SANIC_CUDA_CHECK(ctx, cudaOccupancyMaxActiveClusters(&max_clusters, gemm_rmsnorm_pair_kernel, &cfg));
        SANIC_REQUIRE(ctx, max_clusters >= 1, "gemm_rmsnorm: no SM pair can hold the kernel");
        int pairs = ptiles < max_clusters ? ptiles : max_clusters;
        if (pairs > ctx->sm_count / 2) pairs = ctx->sm_count / 2;
        cfg.gridDim = dim3(2 * pairs);
        if (reg_path) {
            unsigned long long* prof = ctx->gemm_prof;      // set only by sanic_gemm_rmsnorm_pair_profile, for the one launch it makes
            cudaError_t le = prof
                ? cudaLaunchKernelEx(&cfg, gemm_rmsnorm_pair_reg_kernel<true>, map_b, map_y, (const uint16_t*)p->x, (const uint16_t*)p->gamma, p->y,
                                     (int)p->M, (int)p->N, (int)p->K, (int)p->w_is_nk, p->eps, (int)p->out_dtype, ctx->status_dev,
                                     gamma_bytes, bulk_store, prof)
                : cudaLaunchKernelEx(&cfg, gemm_rmsnorm_pair_reg_kernel<false>, map_b, map_y, (const uint16_t*)p->x, (const uint16_t*)p->gamma, p->y,
                                     (int)p->M, (int)p->N, (int)p->K, (int)p->w_is_nk, p->eps, (int)p->out_dtype, ctx->status_dev,
                                     gamma_bytes, bulk_store, prof);
            if (le != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemm_rmsnorm (pair, registers): ") + cudaGetErrorString(le));
            return SANIC_OK;
        }
        cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_rmsnorm_pair_kernel, map_a, map_b, map_y, (const uint16_t*)p->gamma, p->y, (int)p->M,
                                            (int)p->N, (int)p->K, (int)p->w_is_nk, p->eps, (int)p->out_dtype, ctx->status_dev,
                                            gamma_bytes, bulk_store, prescaled ? 1 : 0);
        if (le != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("gemm_rmsnorm (pair): ") + cudaGetErrorString(le));
        return SANIC_OK;
    }
    const int smem = STAGES * STAGE_BYTES + MAX_K * 2 + (int)sizeof(Shared) + 1024;
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int tiles = ((p->M + BM - 1) / BM) * ((p->N + BN - 1) / BN);
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    gemm_rmsnorm_kernel<<<grid, NTHREADS, smem, st>>>(map_a, map_b, (const uint16_t*)p->gamma, p->y, p->M, p->N, p->K,
                                                      p->w_is_nk, p->eps, p->out_dtype, ctx->status_dev);
    SANIC_LAUNCH_CHECK(ctx, "gemm_rmsnorm");
    return SANIC_OK;
}





// One launch of the pair tile with A through registers with its clock counters on (see the kernel): `out` receives 18
// numbers. The launch is a real one (y is written); it synchronises the stream.
extern "C" int32_t sanic_gemm_rmsnorm_pair_profile(sanic_ctx* ctx, const sanic_gemm_rmsnorm_params* p, void* stream, uint64_t* out) {
    if (!ctx || !p || !out) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    unsigned long long* dev = nullptr;
    SANIC_CUDA_CHECK(ctx, cudaMalloc(&dev, 18 * sizeof(unsigned long long)));
    cudaMemsetAsync(dev, 0, 18 * sizeof(unsigned long long), (cudaStream_t)stream);
    ctx->gemm_prof = dev;
    int32_t rc = sanic_gemm_rmsnorm(ctx, p, stream);
    ctx->gemm_prof = nullptr;
    if (rc == SANIC_OK) rc = sanic_sync(ctx, stream);
    if (rc == SANIC_OK && cudaMemcpy(out, dev, 18 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = sanic_fail(ctx, SANIC_ERR_CUDA, "gemm profile: copy failed");
    cudaFree(dev);
    return rc;
}
