// Schedules over a buffer table: the per-run binding surface and the stateful stepping API.
//
// The reference's emitter hands its runtime a program whose stages name their buffers
// (MetalProgram{stages[{kernel, inputs, output}], inputs, dtypes, buffers[(name, elements)]},
// src/emit_metal.rs:1183-1212); buffers are bound BY NAME on every run (Program::try_run /
// ordered_bindings, src/compile.rs:132-229), a replay wires state feedback as aliases or as two
// graphs that trade buffers (Program::capture, src/compile.rs:820-960), and Graph / StepProgram /
// Machine (src/graph.rs:231-356) allocate the states and expose named outputs.
//
// Here a schedule is the stage list of program.cu plus a buffer table and a relocation list: every
// pointer field of a stage that refers to a table buffer is named by (stage, byte offset of the field
// inside sanic_stage_desc, buffer index, byte offset into the buffer). Binding patches those fields;
// nothing else of a stage changes, so a rebind costs a copy of the stage list, never a recompile.
// All validation happens on the host before any CUDA call, and a schedule compiled with a NULL
// context validates bindings without a device (the refusals are testable anywhere).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <set>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

size_t dtype_bytes(int dtype, size_t elements) {
    switch (dtype) {
        case SANIC_F32: case SANIC_U32: return elements * 4;
        case SANIC_F16: case SANIC_BF16: return elements * 2;
        case SANIC_I4: return (elements + 1) / 2;
        default: return 0;
    }
}
const char* dtype_name(int dtype) {
    switch (dtype) {
        case SANIC_F32: return "f32"; case SANIC_F16: return "f16"; case SANIC_BF16: return "bf16";
        case SANIC_U32: return "u32"; case SANIC_I4: return "i4"; default: return "?";
    }
}
std::string shape_text(const int64_t* shape, int rank) {
    std::string s = "[";
    for (int i = 0; i < rank; ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
    return s + "]";
}

struct Buf {
    std::string name;
    int kind = 0, dtype = 0, rank = 0;
    int64_t shape[SANIC_MAX_AXES] = {0};
    size_t elements() const { size_t n = 1; for (int i = 0; i < rank; ++i) n *= (size_t)shape[i]; return n; }
    size_t bytes() const { return std::max<size_t>(dtype_bytes(dtype, elements()), 4); }
};

}  // namespace

struct sanic_schedule {
    sanic_ctx* ctx = nullptr;
    std::string err;                                 // last error when there is no context to hold it
    std::vector<sanic_stage_desc> stages;
    std::vector<Buf> bufs;
    std::vector<sanic_reloc> relocs;
    std::vector<int> outputs;                        // buffer index per root, in root order
    std::vector<std::pair<int, int>> in_place;       // (root index, input buffer index): the root writes that input's buffer
    // the execute path: scratch owned by the schedule, the patched program of the last binding set
    std::vector<void*> scratch;                      // per buffer; null for inputs
    std::vector<const void*> bound;                  // per buffer: what the cached program was patched with
    sanic_program* prog = nullptr;
};

struct sanic_replay {
    sanic_schedule* sch = nullptr;
    std::vector<sanic_program*> parity;              // one frozen step, or two when feedback swaps buffers
    std::vector<std::vector<void*>> base;            // per parity: the address of every table buffer
    std::vector<void*> owned;                        // scratch and state allocations of this replay
    std::vector<std::pair<std::string, int>> states; // machine: state input name -> buffer index
    std::vector<std::pair<std::string, int>> named_outputs;   // machine: output name -> root index
    int next = 0;
    long steps = 0;
};

namespace {

int32_t fail(sanic_schedule* s, int32_t code, const std::string& msg) {
    s->err = msg;
    if (s->ctx) s->ctx->err = msg;
    return code;
}

int find_input(const sanic_schedule* s, const char* name) {
    if (!name) return -1;
    for (size_t i = 0; i < s->bufs.size(); ++i)
        if (s->bufs[i].kind == SANIC_BUF_INPUT && s->bufs[i].name == name) return (int)i;
    return -1;
}

// Program::ordered_bindings (src/compile.rs:190-229): unknown and duplicate names are refused while the set is read,
// then every declared input must be present with the declared shape and storage.
int32_t ordered_bindings(sanic_schedule* s, const sanic_binding* b, int32_t n, std::vector<const sanic_binding*>& by_buf) {
    by_buf.assign(s->bufs.size(), nullptr);
    if (n > 0 && !b) return fail(s, SANIC_ERR_INVALID, "bindings: null array");
    for (int i = 0; i < n; ++i) {
        const int idx = find_input(s, b[i].name);
        if (idx < 0) return fail(s, SANIC_ERR_UNKNOWN_INPUT, std::string("unknown input `") + (b[i].name ? b[i].name : "(null)") + "`");
        if (by_buf[idx]) return fail(s, SANIC_ERR_DUPLICATE_INPUT, "input `" + s->bufs[idx].name + "` was bound more than once");
        by_buf[idx] = &b[i];
    }
    for (size_t i = 0; i < s->bufs.size(); ++i) {
        const Buf& d = s->bufs[i];
        if (d.kind != SANIC_BUF_INPUT) continue;
        const sanic_binding* v = by_buf[i];
        if (!v) return fail(s, SANIC_ERR_MISSING_INPUT, "missing input `" + d.name + "`");
        bool same = v->rank == d.rank;
        for (int a = 0; same && a < d.rank; ++a) same = v->shape[a] == d.shape[a];
        if (!same)
            return fail(s, SANIC_ERR_SHAPE, "input `" + d.name + "` has shape " + shape_text(v->shape, std::max(0, std::min(v->rank, SANIC_MAX_AXES))) +
                                            "; expected " + shape_text(d.shape, d.rank));
        if (v->dtype != d.dtype)
            return fail(s, SANIC_ERR_DTYPE, "input `" + d.name + "` is stored " + dtype_name(v->dtype) + "; expected " + dtype_name(d.dtype));
        if (!v->dptr) return fail(s, SANIC_ERR_INVALID, "input `" + d.name + "` is bound to a null buffer");
    }
    return SANIC_OK;
}

void patch(std::vector<sanic_stage_desc>& stages, const std::vector<sanic_reloc>& relocs, const std::vector<void*>& base) {
    for (const sanic_reloc& r : relocs) {
        char* field = (char*)&stages[r.stage] + r.field_offset;
        void* p = (char*)base[r.buffer] + r.byte_offset;
        std::memcpy(field, &p, sizeof(void*));
    }
}

int32_t alloc_zeroed(sanic_schedule* s, size_t bytes, void** out) {
    if (!s->ctx) return fail(s, SANIC_ERR_CUDA, "this schedule was compiled without a device: it validates bindings but cannot run");
    sanic_set_device(s->ctx);
    cudaError_t e = cudaMalloc(out, bytes);
    if (e == cudaSuccess) e = cudaMemset(*out, 0, bytes);
    if (e != cudaSuccess) return fail(s, e == cudaErrorMemoryAllocation ? SANIC_ERR_NOMEM : SANIC_ERR_CUDA, std::string("buffer allocation: ") + cudaGetErrorString(e));
    return SANIC_OK;
}

// SANIC_DEBUG (read once, as src/lib.rs:38-46 does): 1 = one line per compiled schedule and captured replay,
// 2 = also one line per replayed step with its device time, 3 = also the stage list once per replay.
// SANIC_NANSCAN=1: after every run or replayed step, every float buffer the runtime owns is scanned for non-finite values
// and the first offender is named in the error (src/compile.rs:1261-1275).
int debug_level() {
    static const int level = [] { const char* e = getenv("SANIC_DEBUG"); return e ? atoi(e) : 0; }();
    return level;
}
bool nan_scan_on() {
    static const bool on = [] { const char* e = getenv("SANIC_NANSCAN"); return e && e[0] != '0'; }();
    return on;
}
const char* op_name(int op) {
    switch (op) {
        case SANIC_OP_GEMV: return "contraction"; case SANIC_OP_DECODE_ATTN: return "online-softmax fold"; case SANIC_OP_ARGMAX: return "extremum index";
        case SANIC_OP_RMSNORM: return "rmsnorm"; case SANIC_OP_EMBED: return "gather"; case SANIC_OP_ROPE_CACHE: return "rope + cache write";
        case SANIC_OP_ADVANCE: return "advance"; case SANIC_OP_GENERIC: return "generated";
        case SANIC_OP_ATTN_FWD: return "online-softmax fold (forward)"; case SANIC_OP_GEMM_RMSNORM: return "deferred-norm contraction";
        case SANIC_OP_ROPE: return "rope"; default: return "?";
    }
}
int32_t nan_scan(sanic_schedule* s, const std::vector<void*>& base, void* stream) {
    for (size_t i = 0; i < s->bufs.size(); ++i) {
        const Buf& d = s->bufs[i];
        if (d.kind != SANIC_BUF_SCRATCH || !base[i] || !(d.dtype == SANIC_F32 || d.dtype == SANIC_BF16 || d.dtype == SANIC_F16)) continue;
        uint32_t bad = 0;
        int32_t rc = sanic_count_nonfinite(s->ctx, base[i], d.elements(), d.dtype, stream, &bad);
        if (rc != SANIC_OK) return rc;
        if (bad) return fail(s, SANIC_ERR_INVALID, "nan scan: buffer `" + d.name + "` holds " + std::to_string(bad) + " non-finite value(s)");
    }
    return SANIC_OK;
}

void fill_view(const Buf& d, void* p, sanic_buffer_view* v) {
    v->dptr = p; v->dtype = d.dtype; v->rank = d.rank; v->bytes = d.bytes();
    for (int a = 0; a < SANIC_MAX_AXES; ++a) v->shape[a] = a < d.rank ? d.shape[a] : 0;
}

void free_replay(sanic_replay* r) {
    if (!r) return;
    for (sanic_program* p : r->parity) if (p) sanic_program_destroy(p);
    if (r->sch && r->sch->ctx) { sanic_set_device(r->sch->ctx); for (void* p : r->owned) cudaFree(p); }
    delete r;
}

thread_local std::string g_compile_error;     // why this thread's last sanic_schedule_compile failed (it returns no handle)
}  // namespace

extern "C" {

int32_t sanic_schedule_compile(sanic_ctx* ctx, const sanic_schedule_desc* d, sanic_schedule** out) {
    if (!out) return SANIC_ERR_INVALID;
    *out = nullptr;
    if (!d) return SANIC_ERR_INVALID;
    sanic_schedule* s = new (std::nothrow) sanic_schedule();
    if (!s) return SANIC_ERR_NOMEM;
    s->ctx = ctx;
    auto bad = [&](int32_t code, const std::string& msg) { if (ctx) ctx->err = msg; g_compile_error = msg; delete s; return code; };
    if (!d->stages || d->n_stages <= 0) return bad(SANIC_ERR_INVALID, "schedule: cannot compile an empty stage list");      // CompileError::EmptyOutputs' sibling
    if (!d->outputs || d->n_outputs <= 0) return bad(SANIC_ERR_INVALID, "schedule: no output roots");                         // CompileError::EmptyOutputs
    if (!d->buffers || d->n_buffers <= 0) return bad(SANIC_ERR_INVALID, "schedule: empty buffer table");
    std::set<std::string> names;
    for (int i = 0; i < d->n_buffers; ++i) {
        const sanic_buffer_decl& b = d->buffers[i];
        Buf x;
        if (!b.name || !*b.name) return bad(SANIC_ERR_INVALID, "schedule: buffer " + std::to_string(i) + " has no name");
        x.name = b.name;
        if (!names.insert(x.name).second) return bad(SANIC_ERR_INVALID, "schedule: buffer name `" + x.name + "` is declared twice");
        if (b.kind != SANIC_BUF_INPUT && b.kind != SANIC_BUF_SCRATCH) return bad(SANIC_ERR_INVALID, "schedule: buffer `" + x.name + "` has an unknown kind");
        if (dtype_bytes(b.dtype, 2) == 0) return bad(SANIC_ERR_DTYPE, "schedule: buffer `" + x.name + "` has an unknown storage width");
        if (b.rank < 0 || b.rank > SANIC_MAX_AXES) return bad(SANIC_ERR_INVALID, "schedule: buffer `" + x.name + "` has more than " + std::to_string(SANIC_MAX_AXES) + " axes");
        for (int a = 0; a < b.rank; ++a) {
            if (b.shape[a] <= 0) return bad(SANIC_ERR_INVALID, "schedule: buffer `" + x.name + "` has a non-positive extent (dynamic shapes are not supported)");
            x.shape[a] = b.shape[a];
        }
        x.kind = b.kind; x.dtype = b.dtype; x.rank = b.rank;
        s->bufs.push_back(x);
    }
    s->stages.assign(d->stages, d->stages + d->n_stages);
    for (int i = 0; i < d->n_stages; ++i) {
        std::string why;
        const int32_t rc = sanic::stage_check(d->stages[i], &why, false);
        if (rc != SANIC_OK) return bad(rc, "schedule: stage " + std::to_string(i) + ": " + why);
    }
    for (int i = 0; i < d->n_relocs; ++i) {
        const sanic_reloc& r = d->relocs[i];
        if (r.stage < 0 || r.stage >= d->n_stages || r.buffer < 0 || r.buffer >= d->n_buffers || r.byte_offset < 0 ||
            r.field_offset < 0 || (size_t)r.field_offset + sizeof(void*) > sizeof(sanic_stage_desc) || r.field_offset % 8 != 0)
            return bad(SANIC_ERR_INVALID, "schedule: relocation " + std::to_string(i) + " is out of range");
        if ((size_t)r.byte_offset >= s->bufs[r.buffer].bytes() && r.byte_offset != 0)
            return bad(SANIC_ERR_INVALID, "schedule: relocation " + std::to_string(i) + " points past the end of `" + s->bufs[r.buffer].name + "`");
        s->relocs.push_back(r);
    }
    for (int i = 0; i < d->n_outputs; ++i) {
        if (d->outputs[i] < 0 || d->outputs[i] >= d->n_buffers) return bad(SANIC_ERR_INVALID, "schedule: output root " + std::to_string(i) + " names no buffer");
        s->outputs.push_back(d->outputs[i]);
    }
    for (int i = 0; i < d->n_in_place; ++i) {
        const int root = d->in_place_root[i], in = d->in_place_input[i];
        if (root < 0 || root >= d->n_outputs || in < 0 || in >= d->n_buffers || s->bufs[in].kind != SANIC_BUF_INPUT)
            return bad(SANIC_ERR_INVALID, "schedule: in-place pair " + std::to_string(i) + " does not name a root and an input");
        const Buf& o = s->bufs[s->outputs[root]];
        const Buf& x = s->bufs[in];
        if (o.dtype != x.dtype || o.rank != x.rank || !std::equal(o.shape, o.shape + o.rank, x.shape))
            return bad(SANIC_ERR_INVALID, "schedule: root " + std::to_string(root) + " cannot overwrite `" + x.name + "`: shape or storage differs");
        s->in_place.push_back({root, in});
    }
    s->scratch.assign(s->bufs.size(), nullptr);
    s->bound.assign(s->bufs.size(), nullptr);
    *out = s;
    return SANIC_OK;
}

int32_t sanic_schedule_destroy(sanic_schedule* s) {
    if (!s) return SANIC_ERR_INVALID;
    if (s->prog) sanic_program_destroy(s->prog);
    if (s->ctx) { sanic_set_device(s->ctx); for (void* p : s->scratch) if (p) cudaFree(p); }
    delete s;
    return SANIC_OK;
}

const char* sanic_schedule_last_error(sanic_schedule* s) { return s ? s->err.c_str() : g_compile_error.c_str(); }

int32_t sanic_schedule_input_count(sanic_schedule* s) {
    if (!s) return -1;
    int n = 0;
    for (const Buf& b : s->bufs) n += b.kind == SANIC_BUF_INPUT;
    return n;
}
const char* sanic_schedule_input_name(sanic_schedule* s, int32_t i) {
    if (!s) return nullptr;
    for (const Buf& b : s->bufs)
        if (b.kind == SANIC_BUF_INPUT && i-- == 0) return b.name.c_str();
    return nullptr;
}
int32_t sanic_schedule_output_count(sanic_schedule* s) { return s ? (int32_t)s->outputs.size() : -1; }

// The checks of Program::try_run without running anything.
int32_t sanic_schedule_check_bindings(sanic_schedule* s, const sanic_binding* b, int32_t n) {
    if (!s) return SANIC_ERR_INVALID;
    std::vector<const sanic_binding*> by_buf;
    return ordered_bindings(s, b, n, by_buf);
}

// Backend::execute (src/compile.rs:101-107): bind by name, run every stage, return the roots in order.
int32_t sanic_schedule_execute(sanic_schedule* s, const sanic_binding* b, int32_t n, void* stream, sanic_buffer_view* outputs,
                               int32_t n_outputs) {
    if (!s) return SANIC_ERR_INVALID;
    std::vector<const sanic_binding*> by_buf;
    int32_t rc = ordered_bindings(s, b, n, by_buf);
    if (rc != SANIC_OK) return rc;
    if (n_outputs < (int32_t)s->outputs.size() && outputs) return fail(s, SANIC_ERR_INVALID, "execute: the output array is shorter than the root list");
    std::vector<void*> base(s->bufs.size(), nullptr);
    for (size_t i = 0; i < s->bufs.size(); ++i)
        if (s->bufs[i].kind == SANIC_BUF_INPUT) base[i] = const_cast<void*>(by_buf[i]->dptr);
    for (size_t i = 0; i < s->bufs.size(); ++i) {
        if (s->bufs[i].kind != SANIC_BUF_SCRATCH) continue;
        bool aliased = false;
        for (auto& ip : s->in_place)
            if (s->outputs[ip.first] == (int)i) { base[i] = base[ip.second]; aliased = true; }
        if (aliased) continue;
        if (!s->scratch[i]) { rc = alloc_zeroed(s, s->bufs[i].bytes(), &s->scratch[i]); if (rc != SANIC_OK) return rc; }
        base[i] = s->scratch[i];
    }
    bool same = s->prog != nullptr;
    for (size_t i = 0; same && i < base.size(); ++i) same = s->bound[i] == base[i];
    if (!same) {
        if (!s->ctx) return fail(s, SANIC_ERR_CUDA, "this schedule was compiled without a device: it validates bindings but cannot run");
        if (s->prog) { sanic_program_destroy(s->prog); s->prog = nullptr; }
        std::vector<sanic_stage_desc> patched = s->stages;
        patch(patched, s->relocs, base);
        rc = sanic_program_create(s->ctx, patched.data(), (int32_t)patched.size(), &s->prog);
        if (rc != SANIC_OK) { s->err = s->ctx->err; return rc; }
        for (size_t i = 0; i < base.size(); ++i) s->bound[i] = base[i];
    }
    rc = sanic_program_run(s->prog, stream);
    if (rc != SANIC_OK) { s->err = s->ctx->err; return rc; }
    if (nan_scan_on()) { rc = nan_scan(s, base, stream); if (rc != SANIC_OK) return rc; }
    if (outputs)
        for (size_t i = 0; i < s->outputs.size(); ++i) fill_view(s->bufs[s->outputs[i]], base[s->outputs[i]], &outputs[i]);
    return SANIC_OK;
}

// Program::capture (src/compile.rs:820-960): validate the bindings like a run, validate every feedback pair
// (output index, input name), make an in-place root and its input ONE buffer, and freeze one step — or two, with
// the fed buffers trading places, when some pair is not in place.
int32_t sanic_schedule_capture(sanic_schedule* s, const sanic_binding* b, int32_t n, const int32_t* fb_output,
                               const char* const* fb_input, int32_t n_feedback, int32_t persistent, void* stream, sanic_replay** out) {
    if (!s || !out) return SANIC_ERR_INVALID;
    *out = nullptr;
    std::vector<const sanic_binding*> by_buf;
    int32_t rc = ordered_bindings(s, b, n, by_buf);
    if (rc != SANIC_OK) return rc;
    std::vector<std::pair<int, int>> swaps, aliases;     // (output buffer, input buffer)
    std::set<int> fed_outputs, fed_inputs;
    for (int i = 0; i < n_feedback; ++i) {
        const int root = fb_output[i];
        if (root < 0 || root >= (int)s->outputs.size())
            return fail(s, SANIC_ERR_FEEDBACK, "output index " + std::to_string(root) + " is out of range (" + std::to_string(s->outputs.size()) + " outputs)");
        const int in = find_input(s, fb_input[i]);
        if (in < 0) return fail(s, SANIC_ERR_FEEDBACK, std::string("program has no input named `") + (fb_input[i] ? fb_input[i] : "(null)") + "`");
        const Buf& o = s->bufs[s->outputs[root]];
        const Buf& x = s->bufs[in];
        if (o.rank != x.rank || !std::equal(o.shape, o.shape + o.rank, x.shape))
            return fail(s, SANIC_ERR_FEEDBACK, "output " + std::to_string(root) + " has shape " + shape_text(o.shape, o.rank) + "; input `" + x.name +
                                               "` expects " + shape_text(x.shape, x.rank));
        if (o.dtype != x.dtype)
            return fail(s, SANIC_ERR_FEEDBACK, "input `" + x.name + "` is " + dtype_name(x.dtype) + "; output " + std::to_string(root) + " is stored " + dtype_name(o.dtype));
        if (!fed_outputs.insert(root).second) return fail(s, SANIC_ERR_FEEDBACK, "output " + std::to_string(root) + " is fed back more than once");
        if (!fed_inputs.insert(in).second) return fail(s, SANIC_ERR_FEEDBACK, "input `" + x.name + "` is fed more than once");
        bool in_place = false;
        for (auto& ip : s->in_place) in_place = in_place || ip.first == root;
        // a root compiled in place already writes its predecessor's buffer: the pair is one buffer, not two that trade roles
        (in_place ? aliases : swaps).push_back({s->outputs[root], in});
    }
    if (!s->ctx) return fail(s, SANIC_ERR_CUDA, "this schedule was compiled without a device: it validates bindings but cannot run");
    sanic_replay* r = new (std::nothrow) sanic_replay();
    if (!r) return SANIC_ERR_NOMEM;
    r->sch = s;
    std::vector<void*> base(s->bufs.size(), nullptr);
    for (size_t i = 0; i < s->bufs.size(); ++i)
        if (s->bufs[i].kind == SANIC_BUF_INPUT) base[i] = const_cast<void*>(by_buf[i]->dptr);
    for (size_t i = 0; i < s->bufs.size(); ++i) {
        if (s->bufs[i].kind != SANIC_BUF_SCRATCH) continue;
        bool aliased = false;
        for (auto& a : aliases) aliased = aliased || a.first == (int)i;
        for (auto& ip : s->in_place)      // an in-place root that is not fed back still writes its input's buffer
            if (s->outputs[ip.first] == (int)i) aliased = true;
        if (aliased) continue;
        void* p = nullptr;
        rc = alloc_zeroed(s, s->bufs[i].bytes(), &p);
        if (rc != SANIC_OK) { free_replay(r); return rc; }
        r->owned.push_back(p);
        base[i] = p;
    }
    for (auto& ip : s->in_place) base[s->outputs[ip.first]] = base[ip.second];
    const int parities = swaps.empty() ? 1 : 2;
    for (int par = 0; par < parities; ++par) {
        std::vector<void*> bufs = base;
        if (par == 1)
            for (auto& sw : swaps) { bufs[sw.first] = base[sw.second]; bufs[sw.second] = base[sw.first]; }
        std::vector<sanic_stage_desc> patched = s->stages;
        patch(patched, s->relocs, bufs);
        sanic_program* p = nullptr;
        rc = sanic_program_create(s->ctx, patched.data(), (int32_t)patched.size(), &p);
        if (rc == SANIC_OK) {
            r->parity.push_back(p);
            rc = persistent ? sanic_program_capture_persistent(p, stream) : sanic_program_capture(p, stream);
        }
        if (rc != SANIC_OK) { s->err = s->ctx->err; free_replay(r); return rc; }
        r->base.push_back(bufs);
    }
    if (debug_level() >= 1)
        fprintf(stderr, "sanic: captured %zu stage(s) over %zu buffer(s) as %d frozen step(s), %d kernel(s) each%s\n", s->stages.size(),
                s->bufs.size(), parities, sanic_program_kernel_count(r->parity[0]), persistent ? " (one cooperative kernel)" : "");
    if (debug_level() >= 3)
        for (size_t i = 0; i < s->stages.size(); ++i)
            fprintf(stderr, "sanic:   stage %3zu  %-20s kind %d%s%s\n", i, op_name(s->stages[i].op), s->stages[i].stage_kind,
                    s->stages[i].op == SANIC_OP_GENERIC ? "  " : "",
                    s->stages[i].op == SANIC_OP_GENERIC ? sanic_generic_kernel_name(s->stages[i].u.generic.kernel) : "");
    *out = r;
    return SANIC_OK;
}

// MetalReplay::step_timed (src/compile.rs:1000-1024): replay the next parity; fed-back outputs are already wired as the
// next step's inputs.
int32_t sanic_replay_step(sanic_replay* r, void* stream, double* gpu_seconds) {
    if (!r || r->parity.empty()) return SANIC_ERR_INVALID;
    const int par = r->next;
    r->next = (par + 1) % (int)r->parity.size();
    double sec = 0.0;
    const bool want = gpu_seconds || debug_level() >= 2;
    int32_t rc = sanic_program_step(r->parity[par], stream, want ? &sec : nullptr);
    if (gpu_seconds) *gpu_seconds = sec;
    if (rc == SANIC_OK) ++r->steps; else r->sch->err = r->sch->ctx->err;
    if (rc == SANIC_OK && debug_level() >= 2)
        fprintf(stderr, "sanic: step %ld (frozen step %d of %zu, %d kernel(s)) %.3f ms on the device\n", r->steps, par, r->parity.size(),
                sanic_program_kernel_count(r->parity[par]), sec * 1e3);
    if (rc == SANIC_OK && nan_scan_on()) rc = nan_scan(r->sch, r->base[par], stream);
    return rc;
}

// One step with a device time per stage (the SANIC_DEBUG=4 path of the reference's replay). State advances.
int32_t sanic_replay_stage_times(sanic_replay* r, void* stream, double* seconds, int32_t cap, int32_t* n_out) {
    if (!r || r->parity.empty()) return SANIC_ERR_INVALID;
    const int par = r->next;
    r->next = (par + 1) % (int)r->parity.size();
    int32_t rc = sanic_program_stage_times(r->parity[par], stream, seconds, cap, n_out);
    if (rc == SANIC_OK) ++r->steps;
    return rc;
}

int32_t sanic_replay_phase_profile(sanic_replay* r, void* stream, double* out, int32_t cap, int32_t* n_out) {
    if (!r || r->parity.empty()) return SANIC_ERR_INVALID;
    const int par = r->next;
    r->next = (par + 1) % (int)r->parity.size();
    int32_t rc = sanic_program_phase_profile(r->parity[par], stream, out, cap, n_out);
    if (rc == SANIC_OK) ++r->steps; else r->sch->err = r->sch->ctx->err;
    return rc;
}

int32_t sanic_replay_kernel_count(sanic_replay* r) { return (r && !r->parity.empty()) ? sanic_program_kernel_count(r->parity[0]) : -1; }
int32_t sanic_replay_parities(sanic_replay* r) { return r ? (int32_t)r->parity.size() : -1; }

// MetalReplay::last_outputs (src/compile.rs:1032-1035): root `index` as of the last completed step.
int32_t sanic_replay_output(sanic_replay* r, int32_t index, sanic_buffer_view* out) {
    if (!r || !out || r->parity.empty()) return SANIC_ERR_INVALID;
    sanic_schedule* s = r->sch;
    if (index < 0 || index >= (int32_t)s->outputs.size()) return fail(s, SANIC_ERR_INVALID, "replay_output: no such root");
    const int n = (int)r->parity.size();
    const int last = (r->next + n - 1) % n;
    fill_view(s->bufs[s->outputs[index]], r->base[last][s->outputs[index]], out);
    return SANIC_OK;
}

int32_t sanic_replay_destroy(sanic_replay* r) {
    if (!r) return SANIC_ERR_INVALID;
    free_replay(r);
    return SANIC_OK;
}

// Graph::compile_for + StepProgram::instantiate (src/graph.rs:231-341): the states are inputs of the schedule whose
// successors are roots. A state declared at another width than the compilation's boundary policy is refused
// (src/graph.rs:236-245). State buffers are allocated here, zeroed, and each state's root feeds the next step's
// input; the caller binds only the non-state inputs.
int32_t sanic_machine_instantiate(sanic_schedule* s, const sanic_state_decl* states, int32_t n_states, int32_t boundary_dtype,
                                  const sanic_binding* b, int32_t n, const char* const* output_names, const int32_t* output_roots,
                                  int32_t n_named, int32_t persistent, void* stream, sanic_replay** out) {
    if (!s || !out) return SANIC_ERR_INVALID;
    *out = nullptr;
    if (n_states > 0 && !states) return fail(s, SANIC_ERR_INVALID, "machine: null state list");
    std::vector<int> state_buf(n_states, -1);
    for (int i = 0; i < n_states; ++i) {
        const int in = find_input(s, states[i].input_name);
        if (in < 0) return fail(s, SANIC_ERR_FEEDBACK, std::string("program has no input named `") + (states[i].input_name ? states[i].input_name : "(null)") + "`");
        if (s->bufs[in].dtype != boundary_dtype && !states[i].pinned)
            return fail(s, SANIC_ERR_UNSUPPORTED, "state `" + s->bufs[in].name + "` is declared " + dtype_name(s->bufs[in].dtype) +
                                                  " but the compilation's policy stores step boundaries as " + dtype_name(boundary_dtype));
        state_buf[i] = in;
    }
    for (int i = 0; i < n_named; ++i)
        if (!output_names[i] || output_roots[i] < 0 || output_roots[i] >= (int32_t)s->outputs.size())
            return fail(s, SANIC_ERR_INVALID, "machine: a named output does not refer to a root");
    // a caller binding names a state: the machine owns the states
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n_states; ++j)
            if (b[i].name && s->bufs[state_buf[j]].name == b[i].name)
                return fail(s, SANIC_ERR_DUPLICATE_INPUT, "input `" + s->bufs[state_buf[j]].name + "` is a state: the machine allocates it");
    if (!s->ctx) {
        // without a device only the checks run: the bindings plus zero-sized stand-ins for the states
        std::vector<sanic_binding> all(b, b + n);
        for (int j = 0; j < n_states; ++j) {
            sanic_binding v{};
            const Buf& d = s->bufs[state_buf[j]];
            v.name = d.name.c_str(); v.dptr = (const void*)0x10; v.dtype = d.dtype; v.rank = d.rank;
            for (int a = 0; a < d.rank; ++a) v.shape[a] = d.shape[a];
            all.push_back(v);
        }
        std::vector<const char*> names;
        std::vector<int32_t> roots;
        for (int j = 0; j < n_states; ++j) { names.push_back(s->bufs[state_buf[j]].name.c_str()); roots.push_back(states[j].root); }
        return sanic_schedule_capture(s, all.data(), (int32_t)all.size(), roots.data(), names.data(), n_states, persistent, stream, out);
    }
    std::vector<void*> state_mem(n_states, nullptr);
    std::vector<sanic_binding> all(b, b + n);
    int32_t rc = SANIC_OK;
    for (int j = 0; j < n_states && rc == SANIC_OK; ++j) {
        const Buf& d = s->bufs[state_buf[j]];
        rc = alloc_zeroed(s, d.bytes(), &state_mem[j]);
        sanic_binding v{};
        v.name = d.name.c_str(); v.dptr = state_mem[j]; v.dtype = d.dtype; v.rank = d.rank;
        for (int a = 0; a < d.rank; ++a) v.shape[a] = d.shape[a];
        all.push_back(v);
    }
    std::vector<const char*> names;
    std::vector<int32_t> roots;
    for (int j = 0; j < n_states; ++j) { names.push_back(s->bufs[state_buf[j]].name.c_str()); roots.push_back(states[j].root); }
    sanic_replay* r = nullptr;
    if (rc == SANIC_OK) rc = sanic_schedule_capture(s, all.data(), (int32_t)all.size(), roots.data(), names.data(), n_states, persistent, stream, &r);
    if (rc != SANIC_OK) {
        sanic_set_device(s->ctx);
        for (void* p : state_mem) if (p) cudaFree(p);
        return rc;
    }
    for (int j = 0; j < n_states; ++j) { r->owned.push_back(state_mem[j]); r->states.push_back({s->bufs[state_buf[j]].name, state_buf[j]}); }
    for (int i = 0; i < n_named; ++i) r->named_outputs.push_back({output_names[i], output_roots[i]});
    *out = r;
    return SANIC_OK;
}

// Machine::output (src/graph.rs:343-356): a named output's buffer as of the last completed step.
int32_t sanic_machine_output(sanic_replay* r, const char* name, sanic_buffer_view* out) {
    if (!r || !name || !out) return SANIC_ERR_INVALID;
    for (auto& no : r->named_outputs)
        if (no.first == name) return sanic_replay_output(r, no.second, out);
    return fail(r->sch, SANIC_ERR_UNKNOWN_INPUT, std::string("no output named `") + name + "`");
}

// The buffer that holds state `name` as the NEXT step will read it (for loading a prefilled cache, or reading it back).
int32_t sanic_machine_state(sanic_replay* r, const char* name, sanic_buffer_view* out) {
    if (!r || !name || !out || r->parity.empty()) return SANIC_ERR_INVALID;
    for (auto& st : r->states)
        if (st.first == name) { fill_view(r->sch->bufs[st.second], r->base[r->next][st.second], out); return SANIC_OK; }
    return fail(r->sch, SANIC_ERR_UNKNOWN_INPUT, std::string("no state named `") + name + "`");
}

}  // extern "C"
