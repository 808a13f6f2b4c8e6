// Online-softmax fold in f32 storage and f32 CUDA-core arithmetic.
//
// One CTA of 256 threads folds a block of BQ = 256 / DV query rows of one (batch, head) over the key axis in
// chunks of 256 keys, so K and V are read once per BQ rows instead of once per row. Per chunk:
//   scores   thread j takes key j of the chunk: one pass over its K row gives the BQ scores (q rows broadcast
//            from shared memory); masked or out-of-range keys lift to the identity (-inf, 0, 0)
//   combine  per row, the chunk maximum (warp shuffles, then the 8 warps through shared memory) is combined into
//            the running (m, l, o) with the carrier's own rule, the -inf guard included (reference
//            src/derive.rs:1700-1713): m' = max(m, c), everything carried so far scales by exp(m - m')
//   values   thread (row, e) adds sum_j exp(s_j - m') * V[j][e] over the chunk (V rows read coalesced across e) and,
//            redundantly across e, sum_j exp(s_j - m') into l
// Chunks are folded left to right, which is the lane_stream x sgs schedule of the reference's cooperative fold
// (src/emit_metal.rs:760-1101, src/plan.rs:434-455) with the CTA as the lane group; project o / l at the end.
//
// When the (row block, batch * head) grid alone would leave SMs idle, the key axis is also split over the CTAs of a
// thread-block cluster (up to 8): CTA z folds the contiguous chunk range [z*n/Z, (z+1)*n/Z), leaves its raw (m, l, o)
// in its own shared memory, and CTA 0 merges the partials in rank order through distributed shared memory with the
// carrier's combine: run_carrier_split (src/interp.rs:597-640) with the cluster as the device, no scratch in HBM.
//
// A tensor-core TF32 contraction has a 10-bit mantissa and cannot hold the 1e-5
// relative bound this path is checked at, so the contraction runs as FP32 FMAs and
// exp / division are the full-precision library routines.
//
// The arithmetic type T is a template parameter. T = float is the default. T = double (sanic_attn_params::accum_dtype
// = SANIC_F64) keeps scores, exponentials, l and o in f64 and rounds once at the store: an output that is a near
// cancellation of its terms (a zero crossing) then still has a PLAIN relative error at f32 rounding level against the
// f64 interpreter, which no f32 accumulation can give (the f32 form is accurate relative to the magnitude of the terms,
// |g - e| / (1 + |e|), the reference's own measure, tests/metal.rs:99-156). At 67 MFLOP (config 1) the f64 pipe is not
// the bound either way.
#include "common.cuh"

namespace {
using namespace sanic;

constexpr int NT = 256;      // threads per CTA = keys per chunk

__device__ __forceinline__ float fma_t(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double fma_t(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ float max_t(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ double max_t(double a, double b) { return fmax(a, b); }
__device__ __forceinline__ float exp_t(float a) { return expf(a); }
__device__ __forceinline__ double exp_t(double a) { return exp(a); }
__device__ __forceinline__ float ld_dsmem(uint32_t addr, float) {
    float v; asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory"); return v;
}
__device__ __forceinline__ double ld_dsmem(uint32_t addr, double) {
    double v; asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(addr) : "memory"); return v;
}

template <int DV, typename T>
__global__ void __launch_bounds__(NT) attn_fwd_f32_kernel(sanic_attn_params p) {
    const T NEG_INF = -(T)INFINITY;
    constexpr int BQ = NT / DV;                   // query rows per CTA
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = blockIdx.x * BQ;
    const int bh = blockIdx.y;
    const int z = blockIdx.z, Z = gridDim.z;      // this CTA's share of the key chunks; the cluster spans z
    const int b = bh / p.q_heads, h = bh % p.q_heads;
    const int hk = h / (p.q_heads / p.kv_heads);
    const int E = p.head_dim, Ev = p.v_dim, S = p.kv_len, L = p.q_len;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* ps = (T*)smem_raw;                 // [BQ][NT] weights exp(s - m') of the current chunk
    T* red = ps + BQ * NT;                // [BQ][8] warp maxima
    T* mrow = red + BQ * 8;               // [BQ] running max
    T* arow = mrow + BQ;                  // [BQ] rescale factor of the current chunk
    T* part = arow + BQ;                  // [BQ][2 + DV] this CTA's raw (m, l, o), read by CTA 0 of the cluster
    float* qs = (float*)(part + BQ * (2 + DV));   // [BQ][E]; every T array above has a multiple of 4 elements
    for (int i = tid; i < BQ * E; i += NT) {
        const int r = i / E, d = i % E;
        qs[i] = (r0 + r < L) ? ((const float*)p.q)[((size_t)bh * L + r0 + r) * E + d] : 0.0f;
    }
    if (tid < BQ) mrow[tid] = NEG_INF;
    __syncthreads();

    const float* K = (const float*)p.k + ((size_t)(b * p.kv_heads + hk) * S) * E;
    const float* V = (const float*)p.v + ((size_t)(b * p.kv_heads + hk) * S) * Ev;

    // Visible key range of each row. A causal / window prefix mask contributes exact zeros outside it, so
    // stopping the stream at the edge is bit-identical (src/emit_metal.rs:442-456).
    auto row_lo = [&](int row) { return (p.window > 0) ? max(0, row - p.window + 1) : 0; };
    auto row_hi = [&](int row) { return (row >= L) ? 0 : ((p.causal || p.window > 0) ? min(S, row + 1) : S); };
    const int last_row = min(r0 + BQ, L) - 1;
    const int j_lo = row_lo(r0), j_hi = row_hi(last_row);        // both are monotone in the row

    const int rq = tid / DV, e = tid % DV;       // the (row, output column) this thread accumulates
    T l = 0, o = 0;

    const int c_first = j_lo / NT, n_chunks = (j_hi > j_lo) ? (j_hi + NT - 1) / NT - c_first : 0;
    const int c_begin = c_first + (z * n_chunks) / Z, c_end = c_first + ((z + 1) * n_chunks) / Z;
    for (int c0 = c_begin * NT; c0 < c_end * NT; c0 += NT) {
        // ── scores of key j against the BQ rows ──
        const int j = c0 + tid;
        {   // the chunk's V rows are read 256 FMAs from now: start them towards L1 (one 128-byte line per request)
            const int n_keys = min(NT, S - c0);
            const char* vb = (const char*)(V + (size_t)c0 * Ev);
            const int lines = (n_keys * Ev * 4 + 127) / 128;
            for (int i = tid; i < lines; i += NT) asm volatile("prefetch.global.L1 [%0];" ::"l"(vb + (size_t)i * 128));
        }
        T sc[BQ];
#pragma unroll
        for (int r = 0; r < BQ; ++r) sc[r] = 0;
        if (j < S) {
            if ((E & 3) == 0) {
                const float4* kr = (const float4*)(K + (size_t)j * E);
                // eight independent 16-byte loads of the key row in flight before their FMAs: one round trip per 32 dims
                for (int d0 = 0; d0 < E / 4; d0 += 8) {
                    float4 kv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) kv[u] = (d0 + u < E / 4) ? __ldg(kr + d0 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (d0 + u < E / 4) {
#pragma unroll
                            for (int r = 0; r < BQ; ++r) {
                                const float4 q = *(const float4*)(qs + r * E + 4 * (d0 + u));
                                sc[r] = fma_t((T)q.x, (T)kv[u].x, sc[r]); sc[r] = fma_t((T)q.y, (T)kv[u].y, sc[r]);
                                sc[r] = fma_t((T)q.z, (T)kv[u].z, sc[r]); sc[r] = fma_t((T)q.w, (T)kv[u].w, sc[r]);
                            }
                        }
                    }
                }
            } else {
                for (int d = 0; d < E; ++d) {
                    const float kv = __ldg(K + (size_t)j * E + d);
#pragma unroll
                    for (int r = 0; r < BQ; ++r) sc[r] = fma_t((T)qs[r * E + d], (T)kv, sc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < BQ; ++r) {
            const int row = r0 + r;
            T s = sc[r] * (T)p.scale;
            if (p.mask && row < L && j < S) s += (T)p.mask[(size_t)row * S + j];
            if (!(j >= row_lo(row) && j < row_hi(row))) s = NEG_INF;      // outside the row's range: the identity
            sc[r] = s;
            T mx = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = max_t(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            if (lane == 0) red[r * 8 + warp] = mx;
        }
        __syncthreads();
        // ── combine the chunk maximum into the running maximum ──
        if (tid < BQ) {
            T cm = red[tid * 8];
#pragma unroll
            for (int w = 1; w < 8; ++w) cm = max_t(cm, red[tid * 8 + w]);
            const T m_old = mrow[tid], m_new = max_t(m_old, cm);
            arow[tid] = (m_old > NEG_INF) ? exp_t(m_old - m_new) : (T)0;     // a side at -inf carries weight 0
            mrow[tid] = m_new;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < BQ; ++r) ps[r * NT + tid] = (sc[r] > NEG_INF) ? exp_t(sc[r] - mrow[r]) : (T)0;
        __syncthreads();
        // ── values: (row rq, column e) ──
        {
            const T alpha = arow[rq];
            o *= alpha; l *= alpha;
            const int n = min(NT, min(j_hi, S) - c0);      // keys of this chunk that exist and any row can see
            const T* pr = ps + rq * NT;
            const float* vr = V + (size_t)c0 * Ev + e;
            if (e < Ev) {
                // 32 independent loads in flight per round trip; weights of masked keys are exact zeros
                for (int jj0 = 0; jj0 < n; jj0 += 32) {
                    float vv[32];
#pragma unroll
                    for (int u = 0; u < 32; ++u) vv[u] = (jj0 + u < n) ? __ldg(vr + (size_t)(jj0 + u) * Ev) : 0.0f;
#pragma unroll
                    for (int u = 0; u < 32; ++u) {
                        const T w = pr[jj0 + u];
                        o = fma_t(w, (T)vv[u], o);
                        l += w;
                    }
                }
            }
        }
        __syncthreads();      // ps, red and arow are rewritten by the next chunk
    }
    if (Z > 1) {
        // partials meet in CTA 0 of the cluster, merged left to right in rank (= chunk) order
        part[rq * (2 + DV) + 2 + e] = o;
        if (e == 0) { part[rq * (2 + DV)] = mrow[rq]; part[rq * (2 + DV) + 1] = l; }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (z == 0) {
            T m = mrow[rq];
            for (int q = 1; q < Z; ++q) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(part + rq * (2 + DV))), "r"(q));
                const T mb = ld_dsmem(remote, T()), lb = ld_dsmem(remote + (uint32_t)sizeof(T), T()),
                        ob = ld_dsmem(remote + (uint32_t)sizeof(T) * (2 + e), T());
                // the derived combine of the ExpShifted pair (src/derive.rs:1700-1713): a side at -inf has weight 0
                const T M = max_t(m, mb);
                const T ra = (m > NEG_INF) ? exp_t(m - M) : (T)0, rb = (mb > NEG_INF) ? exp_t(mb - M) : (T)0;
                l = l * ra + lb * rb; o = o * ra + ob * rb; m = M;
            }
        }
        // the other CTAs' shared memory must outlive CTA 0's reads
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (z != 0) return;
    }
    if (e < Ev && r0 + rq < L) ((float*)p.out)[((size_t)bh * L + r0 + rq) * Ev + e] = (float)(o / l);
}
}  // namespace

extern "C" int32_t sanic_attn_fwd_f32(sanic_ctx* ctx, const sanic_attn_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->q && p->k && p->v && p->out, "attn_fwd_f32: null tensor");
    SANIC_REQUIRE(ctx, p->batch > 0 && p->q_heads > 0 && p->kv_heads > 0 && p->q_heads % p->kv_heads == 0,
                  "attn_fwd_f32: query heads must be a multiple of key/value heads");
    SANIC_REQUIRE(ctx, p->q_len > 0 && p->kv_len > 0, "attn_fwd_f32: empty sequence");
    SANIC_REQUIRE(ctx, p->head_dim > 0 && p->head_dim <= 1024, "attn_fwd_f32: head_dim must be in [1, 1024]");
    SANIC_REQUIRE(ctx, p->v_dim > 0 && p->v_dim <= 128, "attn_fwd_f32: v_dim must be in [1, 128]");
    SANIC_REQUIRE(ctx, p->out_dtype == SANIC_F32, "attn_fwd_f32: output is f32");
    SANIC_REQUIRE(ctx, p->accum_dtype == 0 || p->accum_dtype == SANIC_F32 || p->accum_dtype == SANIC_F64,
                  "attn_fwd_f32: accum_dtype must be 0, SANIC_F32 or SANIC_F64");
    SANIC_REQUIRE(ctx, !(p->causal && p->mask), "attn_fwd_f32: attn_mask and is_causal cannot both be set");
    sanic_set_device(ctx);
    const int dv = p->v_dim <= 32 ? 32 : (p->v_dim <= 64 ? 64 : 128);
    const int bq = NT / dv;
    dim3 grid((p->q_len + bq - 1) / bq, p->batch * p->q_heads), block(NT);
    // split the key axis over a cluster when the grid alone would not give every SM two CTAs
    const long long ctas = (long long)grid.x * grid.y;
    const int chunks = (p->kv_len + NT - 1) / NT;
    int splits = (int)((2LL * ctx->sm_count + ctas - 1) / ctas);
    if (splits > 8) splits = 8;
    if (splits > chunks) splits = chunks;
    if (splits < 1 || grid.y > 65535) splits = 1;
    grid.z = splits;
    const bool f64 = p->accum_dtype == SANIC_F64;
    size_t smem = (size_t)bq * p->head_dim * sizeof(float) +
                  ((size_t)bq * NT + (size_t)bq * 10 + (size_t)bq * (2 + dv)) * (f64 ? sizeof(double) : sizeof(float));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e;
    auto launch = [&](auto kern) -> cudaError_t {
        if (smem > 48 * 1024) {
            cudaError_t a = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (a != cudaSuccess) return a;
        }
        return cudaLaunchKernelEx(&cfg, kern, *p);
    };
    if (dv == 32) e = f64 ? launch(attn_fwd_f32_kernel<32, double>) : launch(attn_fwd_f32_kernel<32, float>);
    else if (dv == 64) e = f64 ? launch(attn_fwd_f32_kernel<64, double>) : launch(attn_fwd_f32_kernel<64, float>);
    else e = f64 ? launch(attn_fwd_f32_kernel<128, double>) : launch(attn_fwd_f32_kernel<128, float>);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("attn_fwd_f32: ") + cudaGetErrorString(e));
    return SANIC_OK;
}
