// Online-softmax fold in f32 storage and f32 CUDA-core arithmetic.
//
// One CTA of 8 warps per query row. The key axis is streamed lane-split (the 256 threads
// take keys j, j+256, ...); each lane keeps its own (m, l, o[Ev]) accumulator in registers,
// the 32 lane accumulators of a warp are merged with a shuffle butterfly and the 8 warp
// accumulators through shared memory, every merge applying the carrier's own combine,
// the -inf guard included (reference src/derive.rs:1700-1713). This is the lane_stream x
// sgs schedule of the reference's cooperative fold (src/emit_metal.rs:760-1101,
// src/plan.rs:434-455), written for 32-wide warps.
//
// A tensor-core TF32 contraction has a 10-bit mantissa and cannot hold the 1e-5
// relative bound this path is checked at, so the contraction runs as FP32 FMAs and
// exp / division are the full-precision library routines.
#include "common.cuh"

namespace {
using namespace sanic;

constexpr int FW = 8;   // warps (simdgroups) per query row

template <int DV>
__global__ void __launch_bounds__(FW * 32) attn_fwd_f32_kernel(sanic_attn_params p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / p.q_heads, h = bh % p.q_heads;
    const int hk = h / (p.q_heads / p.kv_heads);
    const int E = p.head_dim, Ev = p.v_dim, S = p.kv_len, L = p.q_len;

    extern __shared__ float smem[];
    float* qs = smem;                 // [E]
    float* ws = smem + E;             // [FW][DV + 2] warp accumulators
    const float* Q = (const float*)p.q + ((size_t)bh * L + row) * E;
    for (int d = threadIdx.x; d < E; d += FW * 32) qs[d] = Q[d];
    __syncthreads();

    const float* K = (const float*)p.k + ((size_t)(b * p.kv_heads + hk) * S) * E;
    const float* V = (const float*)p.v + ((size_t)(b * p.kv_heads + hk) * S) * Ev;

    // Visible key range. A causal / window prefix mask contributes exact zeros outside
    // it, so stopping the stream at the edge is bit-identical (src/emit_metal.rs:442-456).
    int lo = 0, hi = S;
    if (p.causal) hi = min(S, row + 1);
    if (p.window > 0) { hi = min(S, row + 1); lo = max(0, row - p.window + 1); }

    float m = -INFINITY, l = 0.0f;
    float o[DV];
#pragma unroll
    for (int e = 0; e < DV; ++e) o[e] = 0.0f;

    for (int j = lo + threadIdx.x; j < hi; j += FW * 32) {
        float s = 0.0f;
        if ((E & 3) == 0) {
            const float4* kr = (const float4*)(K + (size_t)j * E);
            for (int d4 = 0; d4 < E / 4; ++d4) {
                float4 kv = kr[d4];
                s = fmaf(qs[4 * d4 + 0], kv.x, s);
                s = fmaf(qs[4 * d4 + 1], kv.y, s);
                s = fmaf(qs[4 * d4 + 2], kv.z, s);
                s = fmaf(qs[4 * d4 + 3], kv.w, s);
            }
        } else {
            for (int d = 0; d < E; ++d) s = fmaf(qs[d], K[(size_t)j * E + d], s);
        }
        s *= p.scale;
        if (p.mask) s += p.mask[(size_t)row * S + j];
        // element lift (s, 1, v) combined into the running accumulator
        float mn = fmaxf(m, s);
        float ra = (m > -INFINITY) ? expf(m - mn) : 0.0f;
        float rb = (s > -INFINITY) ? expf(s - mn) : 0.0f;
        l = l * ra + rb;
        const float* vr = V + (size_t)j * Ev;
#pragma unroll
        for (int e = 0; e < DV; ++e)
            if (e < Ev) o[e] = o[e] * ra + rb * vr[e];
        m = mn;
    }
    // butterfly merge of the lane accumulators with the derived combine
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float mo = __shfl_xor_sync(0xffffffffu, m, off);
        float lo_ = __shfl_xor_sync(0xffffffffu, l, off);
        MloScale sc = mlo_rescale(m, mo);
        l = l * sc.ra + lo_ * sc.rb;
#pragma unroll
        for (int e = 0; e < DV; ++e) {
            float oo = __shfl_xor_sync(0xffffffffu, o[e], off);
            o[e] = o[e] * sc.ra + oo * sc.rb;
        }
        m = sc.m;
    }
    // merge the warp accumulators left to right, then project: o / l
    if (lane == 0) { ws[warp * (DV + 2)] = m; ws[warp * (DV + 2) + 1] = l; }
#pragma unroll
    for (int e = 0; e < DV; ++e)
        if ((e & 31) == lane) ws[warp * (DV + 2) + 2 + e] = o[e];
    __syncthreads();
    if (warp == 0) {
        float* out = (float*)p.out + ((size_t)bh * L + row) * Ev;
        for (int e = lane; e < Ev; e += 32) {
            float mm = ws[0], ll = ws[1], oo = ws[2 + e];
#pragma unroll
            for (int w = 1; w < FW; ++w) {
                MloScale sc = mlo_rescale(mm, ws[w * (DV + 2)]);
                ll = ll * sc.ra + ws[w * (DV + 2) + 1] * sc.rb;
                oo = oo * sc.ra + ws[w * (DV + 2) + 2 + e] * sc.rb;
                mm = sc.m;
            }
            out[e] = oo / ll;
        }
    }
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
    SANIC_REQUIRE(ctx, !(p->causal && p->mask), "attn_fwd_f32: attn_mask and is_causal cannot both be set");
    sanic_set_device(ctx);
    dim3 grid(p->q_len, p->batch * p->q_heads), block(FW * 32);
    const int dv = p->v_dim <= 32 ? 32 : (p->v_dim <= 64 ? 64 : 128);
    size_t smem = ((size_t)p->head_dim + (size_t)FW * (dv + 2)) * sizeof(float);
    if (dv == 32) attn_fwd_f32_kernel<32><<<grid, block, smem, (cudaStream_t)stream>>>(*p);
    else if (dv == 64) attn_fwd_f32_kernel<64><<<grid, block, smem, (cudaStream_t)stream>>>(*p);
    else attn_fwd_f32_kernel<128><<<grid, block, smem, (cudaStream_t)stream>>>(*p);
    SANIC_LAUNCH_CHECK(ctx, "attn_fwd_f32");
    return SANIC_OK;
}
