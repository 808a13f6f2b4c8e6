// Planning facts and the device-level split: the part of the reference's planner this backend owns.
//
// The reference prices schedules with `DeviceSpecs` (hardware numbers fitted per device, src/cost.rs:33-119) and
// describes an intra-kernel split of a fold's streamed axis with `FoldSched` (src/plan.rs:434-476); a carrier whose slot
// kinds all merge out of order may be split at every level (`mergeable_out_of_order`, src/plan.rs:478-488). The multi-device
// decode adds one level above the kernel: a device-level factor on the streamed axis, with the carriers as the exchanged
// state, legal under the same rule and priced with the same roofline plus a fixed exchange latency. In-context timing
// of candidates (the reference's SANIC_TUNE path, src/compile.rs:1348-1630) is `sanic_tune_decode`.
#include <algorithm>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace {
__global__ void empty_kernel(int* sink) { if (sink && threadIdx.x == 9999) *sink = 1; }
}

extern "C" {

// DeviceSpecs::b200(): fitted on this pool's B200s from this library's own measured kernels.
int32_t sanic_specs_b200(sanic_fitted_specs* s) {
    if (!s) return SANIC_ERR_INVALID;
    s->sram_bytes = 232448.0;            // 227 KB of shared memory per resident block
    s->regfile_bytes = 262144.0;         // 64 K 32-bit registers per SM
    s->hbm_bandwidth = 6.45e12;          // copy (read + write); a read-only fold streams 7.0e12 (hbm_read_bandwidth)
    s->hbm_read_bandwidth = 7.0e12;
    s->peak_flops = 1.70e15;             // dense bf16, burst (1.41e15 sustained under the power cap)
    s->launch_overhead = 4.0e-6;         // one more kernel in a captured step: launch, ramp and drain
    s->dtype_bytes = 2.0;                // bf16 boundary policy
    s->compute_dtype = SANIC_F32;
    s->boundary_dtype = SANIC_BF16;
    s->min_blocks = 296.0;               // two resident 128-thread CTAs per SM hide the fold's latency
    // Little's law constant: the weight ring of the single-kernel step (4 x 32 KB x 148 SMs in flight) streams 6.0e12 B/s,
    // the stream-K fold (296 CTAs x 2 tiles x 32 KB) 7.1e12 B/s: 19 MB in flight saturate, i.e. about 2.7 us effective.
    s->mem_latency_s = 2.7e-6;
    s->sm_count = 148;
    s->l2_bytes = 126.0 * 1024 * 1024;
    s->exp_per_clk_per_sm = 13.3;        // ex2.approx, 8 resident warps
    s->sm_clock_hz = 1.965e9;
    s->grid_barrier_s = 1.9e-6;          // device-wide barrier inside the cooperative step, arrival to release
    s->exchange_latency_s = 3.5e-5;      // one carrier exchange among 8 devices: peer stores, flags, the slowest device's skew
    s->link_bandwidth = 7.7e11;          // NVLink, per direction per device (measured peer copy)
    return SANIC_OK;
}

// The same structure with the bandwidth, the exponential rate and the launch overhead measured on this device now.
int32_t sanic_specs_measure(sanic_ctx* ctx, void* stream, sanic_fitted_specs* s) {
    if (!ctx || !s) return SANIC_ERR_INVALID;
    sanic_specs_b200(s);
    s->sm_count = ctx->sm_count;
    s->l2_bytes = (double)ctx->l2_bytes;
    s->min_blocks = 2.0 * ctx->sm_count;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    // read-only sweep of 1 GiB
    void* buf = nullptr;
    const size_t bytes = (size_t)1 << 30;
    SANIC_CUDA_CHECK(ctx, cudaMalloc(&buf, bytes));
    cudaError_t e = cudaMemsetAsync(buf, 0, bytes, st);
    double gbs = 0.0;
    int32_t rc = e == cudaSuccess ? sanic_probe_stream(ctx, buf, bytes, 5, stream, &gbs) : SANIC_ERR_CUDA;
    cudaFree(buf);
    if (rc != SANIC_OK) return rc;
    s->hbm_read_bandwidth = gbs * 1e9;
    double rate = 0.0;
    rc = sanic_probe_sfu(ctx, 8, 0, 100, stream, &rate, nullptr);
    if (rc != SANIC_OK) return rc;
    s->exp_per_clk_per_sm = rate;
    // launch overhead: 256 dependent empty kernels in one captured graph, replayed
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ex = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t cs = nullptr;
    e = cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        for (int i = 0; i < 256; ++i) empty_kernel<<<1, 32, 0, cs>>>(nullptr);
        e = cudaStreamEndCapture(cs, &g);
    }
    if (e == cudaSuccess) e = cudaGraphInstantiate(&ex, g, 0);
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    float best = 1e30f;
    for (int r = 0; r < 4 && e == cudaSuccess; ++r) {
        cudaEventRecord(e0, cs);
        e = cudaGraphLaunch(ex, cs);
        cudaEventRecord(e1, cs);
        if (e == cudaSuccess) e = cudaEventSynchronize(e1);
        float ms = 0.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        if (r > 0 && ms < best) best = ms;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (ex) cudaGraphExecDestroy(ex);
    if (g) cudaGraphDestroy(g);
    if (cs) cudaStreamDestroy(cs);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("specs_measure: ") + cudaGetErrorString(e));
    s->launch_overhead_empty = (double)best * 1e-3 / 256.0;     // the floor: an empty kernel after an empty kernel
    return SANIC_OK;
}

// mergeable_out_of_order (src/plan.rs:478-488): every slot kind this backend knows re-associates.
int32_t sanic_mergeable_out_of_order(const sanic_carrier_desc* c) {
    if (!c || c->n_slots < 1 || c->n_slots > 4) return 0;
    for (int i = 0; i < c->n_slots; ++i) {
        const int k = c->kind[i];
        if (!(k == SANIC_SLOT_PLAIN_ADD || k == SANIC_SLOT_PLAIN_MAX || k == SANIC_SLOT_PLAIN_MIN || k == SANIC_SLOT_EXP_SHIFTED ||
              k == SANIC_SLOT_AT_EXTREMUM))
            return 0;
    }
    return 1;
}

// The chunking of run_carrier_split (src/interp.rs:603): part b of B owns [b*n/B, (b+1)*n/B); B <= n keeps every part non-empty.
int32_t sanic_shard_range(int64_t extent, int32_t part, int32_t parts, int64_t* lo, int64_t* hi) {
    if (!lo || !hi || parts < 1 || part < 0 || part >= parts || extent < parts) return SANIC_ERR_INVALID;
    *lo = (int64_t)part * extent / parts;
    *hi = (int64_t)(part + 1) * extent / parts;
    return SANIC_OK;
}

// Price a fold of `points` outputs in `streams` independent operand streams (points of one stream share its operands)
// over a streamed axis of `stream_extent` steps, `bytes_per_step` bytes and `flops_per_step` flops per step summed over
// all streams, for every device count in
// {1, 2, 4, 8} up to max_devices, and return the cheapest: max(bytes / bandwidth, flops / peak, Little's-law floor) +
// launch overhead, plus for d > 1 the exchange: fixed latency + (d - 1) carriers over the link.
int32_t sanic_plan_fold(const sanic_fitted_specs* s, const sanic_carrier_desc* carrier, int64_t points, int64_t streams,
                        int64_t stream_extent, double bytes_per_step, double flops_per_step, int32_t carrier_floats_per_point,
                        int32_t max_devices, sanic_fold_plan* out) {
    if (!s || !carrier || !out || points < 1 || streams < 1 || stream_extent < 1 || max_devices < 1) return SANIC_ERR_INVALID;
    const bool splittable = sanic_mergeable_out_of_order(carrier) != 0;
    sanic_fold_plan best{};
    best.seconds = 1e300;
    for (int d = 1; d <= max_devices && d <= 8; d *= 2) {
        if (d > 1 && (!splittable || stream_extent < d)) break;
        const double steps = (double)stream_extent / d;
        const double bytes = steps * bytes_per_step, flops = steps * flops_per_step;
        // resident CTAs of the stream-K fold; a short axis cannot fill them (a CTA folds whole 64-step tiles)
        const double ctas = std::min(s->min_blocks, std::max(1.0, std::ceil(steps / 64.0) * (double)streams));
        const double in_flight = ctas * 2.0 * 32768.0;
        const double bw = std::min(s->hbm_read_bandwidth, in_flight / s->mem_latency_s);
        sanic_fold_plan p{};
        p.devices = d;
        p.ctas = (int32_t)ctas;
        p.warps = 4; p.lanes = 32;
        p.hbm_seconds = bytes / bw;
        p.flop_seconds = flops / s->peak_flops;
        p.launch_seconds = s->launch_overhead;
        p.exchange_seconds = d > 1 ? s->exchange_latency_s + (double)(d - 1) * points * carrier_floats_per_point * 4.0 / s->link_bandwidth : 0.0;
        p.seconds = std::max(p.hbm_seconds, p.flop_seconds) + p.launch_seconds + p.exchange_seconds;
        if (p.seconds < best.seconds) best = p;
    }
    *out = best;
    return SANIC_OK;
}

// In-context timing of the decode fold's schedule candidates on the caller's own buffers: candidates[i] > 0 is that many
// fixed chunks per (batch, kv head), 0 is the stream-K form. p->partials must hold the scratch of the largest candidate
// (and of sanic_attn_decode_streamk_slots() when 0 is among them). seconds[i] receives the best of `repeats` launches.
int32_t sanic_tune_decode(sanic_ctx* ctx, const sanic_decode_params* p, const int32_t* candidates, int32_t n, int32_t repeats,
                          void* stream, int32_t* best_index, double* seconds) {
    if (!ctx || !p || !candidates || n < 1 || !best_index) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, repeats >= 1 && repeats <= 100, "tune_decode: 1..100 repeats");
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    SANIC_CUDA_CHECK(ctx, cudaEventCreate(&e0));
    SANIC_CUDA_CHECK(ctx, cudaEventCreate(&e1));
    int32_t rc = SANIC_OK;
    double best = 1e300;
    *best_index = -1;
    const size_t max_scratch = sanic_attn_decode_scratch_bytes(p->batch, p->q_heads, p->head_dim, p->n_splits);
    for (int i = 0; i < n && rc == SANIC_OK; ++i) {
        sanic_decode_params q = *p;
        const bool sk = candidates[i] == 0;
        q.n_splits = sk ? sanic_attn_decode_streamk_slots(ctx, p->batch, p->kv_heads, p->head_dim) : candidates[i];
        if (q.n_splits < 1 || sanic_attn_decode_scratch_bytes(q.batch, q.q_heads, q.head_dim, q.n_splits) > max_scratch) {
            rc = sanic_fail(ctx, SANIC_ERR_INVALID, "tune_decode: p->n_splits must be the largest candidate (it sizes the scratch)");
            break;
        }
        // the ticket counters sit behind the partials of THIS candidate's layout: clear them
        const size_t off = (size_t)q.batch * q.q_heads * q.n_splits * (q.head_dim + 2);
        cudaMemsetAsync(q.partials + off, 0, (size_t)q.batch * q.q_heads * sizeof(int), st);
        double t_best = 1e300;
        for (int r = 0; r < repeats + 1 && rc == SANIC_OK; ++r) {
            cudaEventRecord(e0, st);
            rc = sk ? sanic_attn_decode_streamk(ctx, &q, stream) : sanic_attn_decode_splitkv(ctx, &q, stream);
            cudaEventRecord(e1, st);
            if (rc == SANIC_OK && cudaEventSynchronize(e1) != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, "tune_decode: a candidate failed");
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, e0, e1);
            if (r > 0) t_best = std::min(t_best, (double)ms * 1e-3);
        }
        if (seconds) seconds[i] = t_best;
        if (t_best < best) { best = t_best; *best_index = i; }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

}  // extern "C"
