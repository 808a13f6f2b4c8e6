// Launch lists and their frozen replays: the stateful-stepping half of the runtime.
//
// A program is the ordered stage list the emitter produced for one schedule
// (reference src/partition.rs:101-127). `run` launches each stage on the caller's
// stream (Backend::execute, src/compile.rs:101-107). `capture` freezes the list into a
// CUDA graph and `step` replays it, which is what MetalDevice::capture /
// run_graph_timed do with a pre-encoded command buffer (src/metal.rs:634-705). State
// that changes between steps (position, tokens, caches) lives in device buffers the
// stages read through pointers, so a replay needs no host writes.
#include <new>
#include <vector>

#include "common.cuh"
#include "decode_step.cuh"

struct sanic_program {
    sanic_ctx* ctx = nullptr;
    std::vector<sanic_stage_desc> stages;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int kernels = 0;          // kernels one run of the launch list starts
    int step_kernels = 0;     // kernels one replay of the captured step starts
    sanic::step::Plan* plan = nullptr;   // the persistent single-kernel form of the step, when the list allows it
};

namespace sanic {
// Structure checks of one stage that need no device: stage kind against op, op against the carrier's kernel family, leaf
// storage against the weight buffer. Shared by program creation and by schedule compilation (which may run without a context,
// and before any buffer is bound: `pointers` = false leaves the fields a binding fills out of the check).
int32_t stage_check(const sanic_stage_desc& s, std::string* why, bool pointers) {
    auto fail = [&](int32_t code, const char* msg) { if (why) *why = msg; return code; };
    if (s.op == SANIC_OP_GENERIC) {
        // a compiled fallback kernel stands for any stage kind: a carrier no specialised kernel matches, a cone, a gather
        if (s.stage_kind != SANIC_STAGE_FUSED && s.stage_kind != SANIC_STAGE_ELEMENTWISE && s.stage_kind != SANIC_STAGE_GATHER)
            return fail(SANIC_ERR_INVALID, "program: unknown stage kind");
        if (!s.u.generic.kernel || (pointers && !s.u.generic.out) || s.u.generic.n_buffers < 0 || s.u.generic.n_buffers > 16)
            return fail(SANIC_ERR_INVALID, "program: a generic stage needs a compiled kernel, its buffers and an output");
        return SANIC_OK;
    }
    if (s.stage_kind == SANIC_STAGE_FUSED) {
        int32_t family = 0;
        int32_t rc = sanic_emit_select(&s.carrier, &family);
        if (rc != SANIC_OK) return fail(rc, "program: no kernel for this carrier structure");
        bool ok = (s.op == SANIC_OP_GEMV && (family == SANIC_KERNEL_PLAIN_CONTRACTION ||
                                            family == SANIC_KERNEL_GROUPED_I4_CONTRACTION)) ||
                  (s.op == SANIC_OP_DECODE_ATTN && family == SANIC_KERNEL_ONLINE_SOFTMAX_FOLD) ||
                  (s.op == SANIC_OP_ARGMAX && family == SANIC_KERNEL_EXTREMUM_INDEX) ||
                  (s.op == SANIC_OP_ATTN_FWD && family == SANIC_KERNEL_ONLINE_SOFTMAX_FOLD) ||
                  (s.op == SANIC_OP_GEMM_RMSNORM && family == SANIC_KERNEL_DEFERRED_NORM_CONTRACTION);
        if (!ok) return fail(SANIC_ERR_UNSUPPORTED, "program: stage op does not match its carrier");
        if (s.op == SANIC_OP_GEMV) {
            bool i4 = s.u.gemv.weight_dtype == SANIC_I4;
            if (i4 != (family == SANIC_KERNEL_GROUPED_I4_CONTRACTION))
                return fail(SANIC_ERR_DTYPE, "program: leaf storage does not match the weight buffer");
        }
    } else if (s.stage_kind == SANIC_STAGE_ELEMENTWISE) {
        if (!(s.op == SANIC_OP_RMSNORM || s.op == SANIC_OP_ROPE_CACHE || s.op == SANIC_OP_ADVANCE || s.op == SANIC_OP_ROPE))
            return fail(SANIC_ERR_UNSUPPORTED, "program: not an elementwise stage");
    } else if (s.stage_kind == SANIC_STAGE_GATHER) {
        if (s.op != SANIC_OP_EMBED) return fail(SANIC_ERR_UNSUPPORTED, "program: not a gather stage");
    } else {
        return fail(SANIC_ERR_INVALID, "program: unknown stage kind");
    }
    return SANIC_OK;
}
}  // namespace sanic

namespace {
int32_t check_stage(sanic_ctx* ctx, const sanic_stage_desc& s) {
    std::string why;
    const int32_t rc = sanic::stage_check(s, &why, true);
    return rc == SANIC_OK ? rc : sanic_fail(ctx, rc, why);
}
int kernels_of(const sanic_stage_desc& s) { return s.op == SANIC_OP_ARGMAX ? 2 : 1; }

int32_t run_stage(sanic_ctx* ctx, const sanic_stage_desc& s, void* stream) {
    switch (s.op) {
        case SANIC_OP_GEMV: return sanic_gemv(ctx, &s.u.gemv, stream);
        case SANIC_OP_DECODE_ATTN: return sanic_attn_decode_splitkv(ctx, &s.u.decode, stream);
        case SANIC_OP_ARGMAX:
            return sanic_argmax(ctx, s.u.argmax.x, s.u.argmax.rows, s.u.argmax.n, s.u.argmax.out, s.u.argmax.scratch, stream);
        case SANIC_OP_RMSNORM:
            return sanic_rmsnorm(ctx, s.u.rmsnorm.x, s.u.rmsnorm.gamma, s.u.rmsnorm.rows, s.u.rmsnorm.n, s.u.rmsnorm.eps,
                                 s.u.rmsnorm.out, stream);
        case SANIC_OP_EMBED:
            if (s.u.embed.table_dtype == SANIC_I4)
                return sanic_embed_gather_w4(ctx, s.u.embed.table, s.u.embed.scales, s.u.embed.tokens, s.u.embed.batch,
                                             s.u.embed.hidden, s.u.embed.vocab, s.u.embed.group, s.u.embed.out, stream);
            return sanic_embed_gather(ctx, s.u.embed.table, s.u.embed.tokens, s.u.embed.batch, s.u.embed.hidden,
                                      s.u.embed.vocab, s.u.embed.out, stream);
        case SANIC_OP_ROPE_CACHE: return sanic_rope_cache_write(ctx, &s.u.rope_cache, stream);
        case SANIC_OP_ADVANCE: return sanic_advance_position(ctx, s.u.advance.position, stream);
        case SANIC_OP_ATTN_FWD:
            if (s.u.attn.storage == SANIC_BF16) return sanic_attn_fwd_bf16(ctx, &s.u.attn.p, stream);
            if (s.u.attn.storage == SANIC_F32) return sanic_attn_fwd_f32(ctx, &s.u.attn.p, stream);
            return sanic_fail(ctx, SANIC_ERR_DTYPE, "program: attention operands are stored as f32 or bf16");
        case SANIC_OP_GEMM_RMSNORM: return sanic_gemm_rmsnorm(ctx, &s.u.gemm, stream);
        case SANIC_OP_ROPE:
            return sanic_rope_bf16(ctx, s.u.rope.x, s.u.rope.out, s.u.rope.rows, s.u.rope.seq, s.u.rope.head_dim, s.u.rope.table,
                                   s.u.rope.pos0, stream);
        case SANIC_OP_GENERIC:
            return sanic_generic_launch(ctx, s.u.generic.kernel, s.u.generic.buffers, s.u.generic.n_buffers, s.u.generic.out, stream);
        default: return sanic_fail(ctx, SANIC_ERR_INVALID, "program: unknown op");
    }
}
}  // namespace

extern "C" {

int32_t sanic_program_create(sanic_ctx* ctx, const sanic_stage_desc* stages, int32_t n_stages, sanic_program** out) {
    if (!ctx || !out) return SANIC_ERR_INVALID;
    *out = nullptr;
    SANIC_REQUIRE(ctx, stages && n_stages > 0, "program: cannot compile an empty stage list");
    sanic_program* p = new (std::nothrow) sanic_program();
    if (!p) return SANIC_ERR_NOMEM;
    p->ctx = ctx;
    for (int i = 0; i < n_stages; ++i) {
        int32_t rc = check_stage(ctx, stages[i]);
        if (rc != SANIC_OK) { delete p; return rc; }
        p->stages.push_back(stages[i]);
        p->kernels += kernels_of(stages[i]);
    }
    *out = p;
    return SANIC_OK;
}

int32_t sanic_program_destroy(sanic_program* p) {
    if (!p) return SANIC_ERR_INVALID;
    sanic_set_device(p->ctx);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    if (p->ev0) cudaEventDestroy(p->ev0);
    if (p->ev1) cudaEventDestroy(p->ev1);
    sanic::step::destroy(p->plan);
    delete p;
    return SANIC_OK;
}

int32_t sanic_program_kernel_count(sanic_program* p) { return p ? (p->exec ? p->step_kernels : p->kernels) : -1; }

int32_t sanic_program_run(sanic_program* p, void* stream) {
    if (!p) return SANIC_ERR_INVALID;
    for (const sanic_stage_desc& s : p->stages) {
        int32_t rc = run_stage(p->ctx, s, stream);
        if (rc != SANIC_OK) return rc;
    }
    return SANIC_OK;
}

static int32_t capture_impl(sanic_program* p, void* stream, bool want_persistent) {
    sanic_ctx* ctx = p->ctx;
    SANIC_REQUIRE(ctx, stream != nullptr, "program_capture: needs a non-default stream");
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (p->exec) { cudaGraphExecDestroy(p->exec); p->exec = nullptr; }
    if (p->graph) { cudaGraphDestroy(p->graph); p->graph = nullptr; }
    if (p->plan) { sanic::step::destroy(p->plan); p->plan = nullptr; }
    // The tail of a decode step is a contraction over the whole vocabulary and the token choice. Where sanic_gemv has a faster
    // stand-alone kernel for that contraction than the step kernel's phase (int4 weights at small batch), the cooperative
    // kernel ends in front of it and the tail stays a launch list behind it.
    size_t split = p->stages.size();
    if (want_persistent) {
        for (size_t i = p->stages.size(); i-- > 1;) {
            if (p->stages[i].op != SANIC_OP_GEMV) continue;
            if (sanic::gemv::rows_form_applies(ctx, p->stages[i].u.gemv)) split = i;
            break;
        }
        const std::vector<sanic_stage_desc> head(p->stages.begin(), p->stages.begin() + split);
        int32_t brc = sanic::step::build(ctx, head, &p->plan);
        if (brc != SANIC_OK) return brc == SANIC_ERR_UNSUPPORTED
                                        ? sanic_fail(ctx, brc, "program_capture_persistent: a stage of this list has no phase in the persistent kernel")
                                        : brc;
    }
    SANIC_CUDA_CHECK(ctx, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int32_t rc = p->plan ? sanic::step::launch(ctx, p->plan, st) : sanic_program_run(p, stream);
    p->step_kernels = p->plan ? 1 : p->kernels;
    for (size_t i = split; p->plan && rc == SANIC_OK && i < p->stages.size(); ++i) {
        rc = run_stage(ctx, p->stages[i], stream);
        p->step_kernels += kernels_of(p->stages[i]);
    }
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (rc != SANIC_OK) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("program_capture: ") + cudaGetErrorString(e));
    p->graph = g;
    SANIC_CUDA_CHECK(ctx, cudaGraphInstantiate(&p->exec, p->graph, 0));
    if (!p->ev0) {
        SANIC_CUDA_CHECK(ctx, cudaEventCreate(&p->ev0));
        SANIC_CUDA_CHECK(ctx, cudaEventCreate(&p->ev1));
    }
    return SANIC_OK;
}

int32_t sanic_program_capture(sanic_program* p, void* stream) {
    if (!p) return SANIC_ERR_INVALID;
    return capture_impl(p, stream, false);
}

// The same replay as ONE cooperative kernel that walks the stage list with grid-wide barriers (decode_step.cu).
int32_t sanic_program_capture_persistent(sanic_program* p, void* stream) {
    if (!p) return SANIC_ERR_INVALID;
    return capture_impl(p, stream, true);
}

// A replay whose launch fails returns an error: the step's writes are untrustworthy and a
// decode loop must not continue on them (reference src/metal.rs:666-705).
int32_t sanic_program_step(sanic_program* p, void* stream, double* gpu_seconds) {
    if (!p) return SANIC_ERR_INVALID;
    sanic_ctx* ctx = p->ctx;
    SANIC_REQUIRE(ctx, p->exec != nullptr, "program_step: capture the program first");
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (gpu_seconds) SANIC_CUDA_CHECK(ctx, cudaEventRecord(p->ev0, st));
    SANIC_CUDA_CHECK(ctx, cudaGraphLaunch(p->exec, st));
    if (gpu_seconds) {
        SANIC_CUDA_CHECK(ctx, cudaEventRecord(p->ev1, st));
        SANIC_CUDA_CHECK(ctx, cudaEventSynchronize(p->ev1));
        float ms = 0.0f;
        SANIC_CUDA_CHECK(ctx, cudaEventElapsedTime(&ms, p->ev0, p->ev1));
        *gpu_seconds = (double)ms * 1e-3;
    }
    return SANIC_OK;
}

// One step with a device time per stage (reference MetalDevice::run_kernel_timed, src/metal.rs:431-447: per-kernel
// times measured inside the one submission). A program captured in its persistent form reports the clock stamps
// its kernel takes at every phase boundary (argmax counts as two phases); otherwise the stages run from the launch
// list with an event between them. The step is a real one: state advances.
int32_t sanic_program_stage_times(sanic_program* p, void* stream, double* seconds, int32_t cap, int32_t* n_out) {
    if (!p || !seconds || !n_out || cap < 0) return SANIC_ERR_INVALID;
    sanic_ctx* ctx = p->ctx;
    sanic_set_device(ctx);
    cudaStream_t st = (cudaStream_t)stream;
    if (p->exec && p->plan) {
        SANIC_CUDA_CHECK(ctx, cudaGraphLaunch(p->exec, st));
        SANIC_CUDA_CHECK(ctx, cudaStreamSynchronize(st));
        *n_out = sanic::step::phase_times(ctx, p->plan, seconds, cap);
        return SANIC_OK;
    }
    const int n = (int)p->stages.size();
    std::vector<cudaEvent_t> ev(n + 1, nullptr);
    int32_t rc = SANIC_OK;
    for (int i = 0; i <= n && rc == SANIC_OK; ++i)
        if (cudaEventCreate(&ev[i]) != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, "program_stage_times: cannot create events");
    if (rc == SANIC_OK && cudaEventRecord(ev[0], st) != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, "program_stage_times: event record failed");
    for (int i = 0; i < n && rc == SANIC_OK; ++i) {
        rc = run_stage(ctx, p->stages[i], stream);
        if (rc == SANIC_OK && cudaEventRecord(ev[i + 1], st) != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, "program_stage_times: event record failed");
    }
    if (rc == SANIC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = sanic_fail(ctx, SANIC_ERR_CUDA, "program_stage_times: the step failed");
    if (rc == SANIC_OK) {
        *n_out = std::min<int32_t>(cap, n);
        for (int i = 0; i < *n_out; ++i) {
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
            seconds[i] = (double)ms * 1e-3;
        }
    }
    for (cudaEvent_t e : ev) if (e) cudaEventDestroy(e);
    return rc;
}

// A finer view of one step of a program captured in its single-kernel form: per phase, seconds from the phase's start to
// (0) activations staged, (1) last contraction done, (2) sums and epilogue done, (3) the grid barrier released, as one
// block saw them. `out` receives 4 * min(cap, phases) numbers. The step is a real one. Synchronises `stream`.
int32_t sanic_program_phase_profile(sanic_program* p, void* stream, double* out, int32_t cap, int32_t* n_out) {
    if (!p || !out || !n_out || cap < 0) return SANIC_ERR_INVALID;
    sanic_ctx* ctx = p->ctx;
    SANIC_REQUIRE(ctx, p->exec && p->plan, "program_phase_profile: capture the program in its single-kernel form first");
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaGraphLaunch(p->exec, (cudaStream_t)stream));
    SANIC_CUDA_CHECK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    *n_out = sanic::step::phase_profile(ctx, p->plan, out, cap);
    return SANIC_OK;
}

}  // extern "C"
