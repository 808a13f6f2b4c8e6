// One decode step as one persistent, cooperatively launched kernel.
//
// A captured launch list pays a fixed cost per kernel (launch, ramp-up, drain) that is several times
// the HBM time of a decode-step stage: a 2048x2048 bf16 projection is 8 MB, 1.3 us of bandwidth. Here
// the stage list (reference src/partition.rs:101-127) is lowered once into a table of phases; a grid of
// co-resident CTAs walks the table, each phase strided over the CTAs, with a grid-wide barrier where the
// launch list had a kernel boundary. While a CTA waits at the barrier, the weights of its first tile of
// the next phase are already on their way into L2, so HBM keeps streaming across the boundary.
//
// The phases reuse the device bodies of the stand-alone kernels (gemv_body.cuh, attn_decode_body.cuh), so
// both paths compute bit-identical results. Data written in one phase and read in a later one crosses SMs
// inside one kernel: those reads go to L2 (ld.global.cg), never through the non-coherent L1.
//
// The barrier is a monotonic arrival counter (cleared on the stream before the launch). Every spin is
// bounded: a CTA that gives up raises the abort word, records a code in the context's status word and
// leaves; the others see the abort word or run out of spins themselves, so the kernel always ends.
#include "decode_step.cuh"

#include <new>

#include "attn_decode_body.cuh"
#include "gemv_body.cuh"

namespace sanic {
namespace step {
namespace {

enum { PH_GEMV = 1, PH_DECODE, PH_EMBED, PH_RMSNORM, PH_ARGMAX_PART, PH_ARGMAX_FINAL, PH_ADVANCE };
constexpr int THREADS = 256;
constexpr int AMAX_CHUNKS = 128;
constexpr unsigned BARRIER_SPIN_LIMIT = 1u << 22;

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

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// bar[0]: arrivals so far in this launch, bar[1]: abort word
__device__ __forceinline__ bool grid_barrier(unsigned* bar, unsigned target, int* err, int* s_ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        int ok = 1;
        unsigned spins = 0;
        while (ld_acquire(bar) < target) {
            if ((++spins & 63u) == 0 && ld_acquire(bar + 1) != 0) { ok = 0; break; }
            if (spins > BARRIER_SPIN_LIMIT) { atomicExch(bar + 1, 1u); atomicCAS(err, 0, 31); ok = 0; break; }
        }
        __threadfence();
        *s_ok = ok;
    }
    __syncthreads();
    return *s_ok != 0;
}

// Each phase body is its own function so that its registers are allocated apart from the other bodies'.
template <bool W4, int NT, bool DUAL, bool NORM>
__device__ __noinline__ void run_gemv(const Phase& P, float* scratch) {
    if (NORM) gemv::row_norms<true>(P.fz, P.batch, P.K, scratch);   // once per phase, not per tile
    for (int blk = blockIdx.x; blk < P.n_blocks; blk += gridDim.x) {
        gemv::gemv_tile<W4, NT, DUAL, NORM, true>(P.x, P.batch, P.K, P.segs, P.n_segments, P.out_dtype, P.epilogue, P.residual,
                                           P.fz, 1, blk, false, scratch);
        __syncthreads();   // the scratch is reused by the next tile
    }
}

template <bool VT>
__device__ __noinline__ void run_decode(const Phase& P, int per_b, unsigned char* dyn, int tid) {
    for (int it = blockIdx.x; it < P.n_blocks; it += gridDim.x) {
        const int b = it / per_b, hk = (it % per_b) / P.dec.n_splits, split = it % P.dec.n_splits;
        decode::attn_decode_tile<64, VT>(P.dec, P.counters, split, hk, b, dyn, tid, false, 1);
        decode::tile_sync(1);
    }
}

// Ask L2 for the weights of this CTA's first tile of a contraction phase (16 rows x K per matrix).
__device__ __forceinline__ void prefetch_gemv(const Phase& P) {
    if ((int)blockIdx.x >= P.n_blocks) return;
    const bool w4 = P.variant & 1, dual = (P.variant & 4) != 0;
    const int gtile = blockIdx.x;
    int seg = 0;
    if (!dual) {
        if (P.n_segments > 1 && gtile >= P.segs.tile_begin[1]) seg = 1;
        if (P.n_segments > 2 && gtile >= P.segs.tile_begin[2]) seg = 2;
    }
    const int tile = gtile - P.segs.tile_begin[seg];
    const size_t row_bytes = w4 ? (size_t)P.K / 2 : (size_t)P.K * 2;
    const int lines = (int)((row_bytes + 127) / 128);
    for (int mI = 0; mI < (dual ? 2 : 1); ++mI) {
        const char* wbase = (const char*)P.segs.w[dual ? mI : seg];
        for (int i = threadIdx.x; i < 16 * lines; i += THREADS) {
            const int r = i / lines, ln = i % lines;
            size_t wrow;
            if (P.epilogue == SANIC_EPI_ROPE_CACHE) {   // rows 8*sub + r and their rotate-half partners
                const int tph = P.fz.head_dim / 16, head = tile / tph, sub = tile % tph;
                wrow = (size_t)head * P.fz.head_dim + 8 * sub + (r & 7) + (r >= 8 ? P.fz.head_dim / 2 : 0);
            } else {
                wrow = (size_t)tile * 16 + r;
            }
            asm volatile("prefetch.global.L2 [%0];" ::"l"(wbase + wrow * row_bytes + (size_t)ln * 128));
        }
    }
}

__device__ __forceinline__ void amax_merge(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}

__global__ void __launch_bounds__(THREADS, 1)
decode_step_kernel(const Phase* __restrict__ phases, int n_phases, unsigned* bar, int* err, unsigned long long* stamps) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ Phase ph[2];
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    constexpr int PW = sizeof(Phase) / 4;
    for (int w = tid; w < PW; w += THREADS) ((int*)&ph[0])[w] = __ldg((const int*)&phases[0] + w);
    __syncthreads();
    // CTA 0 stamps the device clock at every phase boundary (per-stage times inside the one launch)
    if (blockIdx.x == 0 && tid == 0) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); stamps[0] = g; }

    for (int i = 0; i < n_phases; ++i) {
        const Phase& P = ph[i & 1];
        if (i + 1 < n_phases)   // next descriptor: in shared memory by the time the barrier releases
            for (int w = tid; w < PW; w += THREADS) ((int*)&ph[(i + 1) & 1])[w] = __ldg((const int*)&phases[i + 1] + w);

        switch (P.op) {
            case PH_GEMV: {
                float* scratch = (float*)dyn;
                switch (P.variant & 15) {
                    case 0: run_gemv<false, 1, false, false>(P, scratch); break;
                    case 1: run_gemv<true, 1, false, false>(P, scratch); break;
                    case 2: run_gemv<false, 2, false, false>(P, scratch); break;
                    case 3: run_gemv<true, 2, false, false>(P, scratch); break;
                    case 4: run_gemv<false, 1, true, false>(P, scratch); break;
                    case 5: run_gemv<true, 1, true, false>(P, scratch); break;
                    case 6: run_gemv<false, 2, true, false>(P, scratch); break;
                    case 7: run_gemv<true, 2, true, false>(P, scratch); break;
                    case 8: run_gemv<false, 1, false, true>(P, scratch); break;
                    case 9: run_gemv<true, 1, false, true>(P, scratch); break;
                    case 12: run_gemv<false, 1, true, true>(P, scratch); break;
                    case 13: run_gemv<true, 1, true, true>(P, scratch); break;
                    default: break;    // the host never emits other variants
                }
                break;
            }
            case PH_DECODE: {
                // one item = (chunk, kv head, batch) on the first 128 threads; the ring needs the whole dynamic buffer
                const int per_b = P.dec.n_splits * P.dec.kv_heads;
                if (tid < 128) {
                    if (P.variant & 1) run_decode<true>(P, per_b, dyn, tid);
                    else run_decode<false>(P, per_b, dyn, tid);
                }
                break;
            }
            case PH_EMBED: {   // out[b,:] = widen(table[token[b],:])
                const uint16_t* table = (const uint16_t*)P.a;
                const int32_t* tokens = (const int32_t*)P.b;
                float* out = (float*)P.c;
                const int hidden = P.i1, vocab = P.i2;
                for (int b = blockIdx.x; b < P.n_blocks; b += gridDim.x) {
                    int tok = __ldcg(tokens + b);
                    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
                    for (int k = tid; k < hidden; k += THREADS) out[(size_t)b * hidden + k] = bf16_to_f32(table[(size_t)tok * hidden + k]);
                }
                break;
            }
            case PH_RMSNORM: {   // xn = bf16((x * g) / sqrt(sum(x^2) * (1/n) + eps)), fixed summation order
                const float* x = (const float*)P.a;
                const uint16_t* gamma = (const uint16_t*)P.b;
                uint16_t* out = (uint16_t*)P.c;
                const int n = P.i1;
                float* wsum = (float*)dyn;
                for (int row = blockIdx.x; row < P.n_blocks; row += gridDim.x) {
                    const float* xr = x + (size_t)row * n;
                    float ss = 0.0f;
                    for (int k = tid; k < n; k += THREADS) { const float v = __ldcg(xr + k); ss = fmaf(v, v, ss); }
                    ss = warp_sum(ss);
                    if ((tid & 31) == 0) wsum[tid >> 5] = ss;
                    __syncthreads();
                    if (tid == 0) {
                        float tot = 0.0f;
                        for (int w = 0; w < 8; ++w) tot += wsum[w];
                        wsum[8] = sqrtf(tot * (1.0f / (float)n) + P.f0);
                    }
                    __syncthreads();
                    const float den = wsum[8];
                    for (int k = tid; k < n; k += THREADS)
                        out[(size_t)row * n + k] = f32_to_bf16_bits((__ldcg(xr + k) * bf16_to_f32(gamma[k])) / den);
                    __syncthreads();
                }
                break;
            }
            case PH_ARGMAX_PART: {   // (max value, first index) per chunk of a row
                const float* x = (const float*)P.a;
                const int n = P.i1;
                float* sv = (float*)dyn; int* si = (int*)dyn + 8;
                for (int blk = blockIdx.x; blk < P.n_blocks; blk += gridDim.x) {
                    const int row = blk / AMAX_CHUNKS, chunk = blk % AMAX_CHUNKS;
                    const int lo = (int)(((long long)chunk * n) / AMAX_CHUNKS), hi = (int)(((long long)(chunk + 1) * n) / AMAX_CHUNKS);
                    const float* xr = x + (size_t)row * n;
                    float v = -INFINITY; int idx = 0x7FFFFFFF;
                    for (int j = lo + tid; j < hi; j += THREADS) amax_merge(v, idx, __ldcg(xr + j), j);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        float v2 = __shfl_xor_sync(0xffffffffu, v, o); int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
                        amax_merge(v, idx, v2, i2);
                    }
                    if ((tid & 31) == 0) { sv[tid >> 5] = v; si[tid >> 5] = idx; }
                    __syncthreads();
                    if (tid == 0) {
                        for (int w = 1; w < 8; ++w) amax_merge(v, idx, sv[w], si[w]);
                        P.scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2] = v;
                        P.scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2 + 1] = __int_as_float(idx);
                    }
                    __syncthreads();
                }
                break;
            }
            case PH_ARGMAX_FINAL: {
                uint32_t* out = (uint32_t*)P.c;
                float* sv = (float*)dyn; int* si = (int*)dyn + 8;
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
                    __syncthreads();
                    if (tid == 0) {
                        for (int w = 1; w < 8; ++w) amax_merge(v, idx, sv[w], si[w]);
                        out[row] = (idx == 0x7FFFFFFF) ? 0xFFFFFFFFu : (uint32_t)idx;   // the +inf identity saturates to u32::MAX
                    }
                    __syncthreads();
                }
                break;
            }
            case PH_ADVANCE:
                if (blockIdx.x == 0 && tid == 0) *(int32_t*)P.c += 1;
                break;
            default: break;
        }

        if (i + 1 < n_phases) {
            __syncthreads();                          // the next descriptor is complete in shared memory
            const Phase& N = ph[(i + 1) & 1];
            if (N.op == PH_GEMV) prefetch_gemv(N);
            if (!grid_barrier(bar, (unsigned)(i + 1) * gridDim.x, err, &s_ok)) return;
        }
        if (blockIdx.x == 0 && tid == 0) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); stamps[i + 1] = g; }
    }
}

}  // namespace

struct Plan {
    Phase* d_phases = nullptr;
    unsigned* d_bar = nullptr;
    unsigned long long* d_stamps = nullptr;
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
    delete plan;
}

int32_t build(sanic_ctx* ctx, const std::vector<sanic_stage_desc>& stages, Plan** out) {
    *out = nullptr;
    std::vector<Phase> ph;
    size_t smem = 64 * 4;    // pointwise phases
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
                if (norm && wide) return SANIC_ERR_UNSUPPORTED;
                P.op = PH_GEMV; P.n_blocks = tiles;
                P.variant = (w4 ? 1 : 0) | (wide ? 2 : 0) | (dual ? 4 : 0) | (norm ? 8 : 0);
                P.x = (const uint16_t*)g.x; P.batch = g.batch; P.K = g.K; P.n_segments = g.n_segments;
                P.out_dtype = g.out_dtype; P.epilogue = g.epilogue; P.residual = g.residual;
                smem = std::max(smem, (size_t)(wide ? (dual ? gemv::scratch_floats<2, true>() : gemv::scratch_floats<2, false>())
                                                    : (dual ? gemv::scratch_floats<1, true>() : gemv::scratch_floats<1, false>())) * 4);
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
                smem = std::max(smem, (size_t)decode::Cfg<64>::SMEM);
                break;
            }
            case SANIC_OP_EMBED:
                SANIC_REQUIRE(ctx, s.u.embed.table && s.u.embed.tokens && s.u.embed.out && s.u.embed.batch > 0, "step: bad embed stage");
                P.op = PH_EMBED; P.n_blocks = s.u.embed.batch;
                P.a = s.u.embed.table; P.b = s.u.embed.tokens; P.c = s.u.embed.out; P.i1 = s.u.embed.hidden; P.i2 = s.u.embed.vocab;
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
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    SANIC_CUDA_CHECK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, THREADS, smem));
    if (per_sm < 1) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "step: the persistent kernel does not fit on an SM");
    int coop = 0;
    SANIC_CUDA_CHECK(ctx, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    if (!coop) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "step: the device has no cooperative launch");
    Plan* plan = new (std::nothrow) Plan();
    if (!plan) return SANIC_ERR_NOMEM;
    plan->n = (int)ph.size();
    plan->grid = ctx->sm_count;     // one block per SM: each phase body may use the whole register file
    plan->smem = smem;
    cudaError_t e = cudaMalloc(&plan->d_phases, ph.size() * sizeof(Phase));
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_bar, 2 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc(&plan->d_stamps, (ph.size() + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(plan->d_stamps, 0, (ph.size() + 1) * sizeof(unsigned long long));
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
    void* args[] = {(void*)&phases_arg, (void*)&n, (void*)&bar, (void*)&err, (void*)&stamps};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)decode_step_kernel, dim3(plan->grid), dim3(THREADS), args, plan->smem, stream);
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

}  // namespace step
}  // namespace sanic
