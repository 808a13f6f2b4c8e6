// The generic emitter: any carrier, given as expression programs, becomes CUDA C text that is compiled at
// run time for sm_100a. This is the fallback for carriers no specialised kernel matches, and the pointwise
// kernel for elementwise cones.
//
// It plays the role of the reference's generated-source kernels (src/emit_metal.rs):
//   scalar fold       one thread per output point, the streamed axis folded serially in registers
//                     (x = leaves, el = into(x), acc = combine(acc, el), then project, optional elementwise
//                     epilogue, narrowed store)                                        :626-736
//   cooperative fold  the streamed axis split over the 32 lanes of a warp, lane partials merged with the
//                     carrier's OWN combine                                            :760-1101
//   pointwise         value per output point                                           :1118-1178
// and of the shared node -> code recursion (src/codegen.rs:283-443): here a node is a postfix program over
// strided loads, coordinates and the closed scalar basis (src/scalar.rs:45-69; Expr, src/derive.rs:96-118).
//
// Arithmetic is f32 in registers, loads and stores are typed (bf16 widen, int4 nibble q+8, bf16 RNE store, u32
// saturating store: src/emit_metal.rs:119-232). A leaf may be a contraction computed in the fold body (sum over an
// inner axis) or a gather (index rounded half away from zero, then bounds-checked: an index out of range reads 0 and
// leaves code 51 in the context's status word). A store may be conditional (the in-place where(c, x, s)).
// Schedules (FoldSched, src/plan.rs:434-488):
//   lanes = 1                one thread per output point.
//   lanes = 32               the streamed axis over the lanes of a warp: lane b of B = min(32, stream) folds the
//                            contiguous chunk [b*n/B, (b+1)*n/B) and the partials merge left to right in lane order, the
//                            chunking and merge order of run_carrier_split (src/interp.rs:597-640), legal for every
//                            associative carrier; `interleave` (lane b takes s = b, b+32, ...: coalesced for a unit
//                            stream stride) needs a carrier that merges out of order (src/plan.rs:481-488).
//   warps = 2..8             the same split over all threads of a block, warp partials merged in warp order through
//                            shared memory.
//   lane_axis                the LAST grid axis over the lanes instead: a warp owns 32 neighbouring output points, a
//                            contracted leaf that does not read that axis is computed once per warp (inner axis over
//                            the lanes, butterfly sum), and with warps > 1 the streamed axis is split over the warps.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <vector>

#include "common.cuh"

namespace {

// ── NVRTC, resolved at run time so that the library has no link-time dependency on it ──
struct Nvrtc {
    void* lib = nullptr;
    nvrtcResult (*create)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    nvrtcResult (*compile)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*cubin_size)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*cubin)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*log_size)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*log)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*destroy)(nvrtcProgram*) = nullptr;
    const char* (*err)(nvrtcResult) = nullptr;
    bool ok = false;
};
Nvrtc& nvrtc() {
    static Nvrtc n = [] {
        Nvrtc r;
        const char* names[] = {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"};
        for (const char* nm : names) {
            r.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
            if (r.lib) break;
        }
        if (!r.lib) return r;
        r.create = (decltype(r.create))dlsym(r.lib, "nvrtcCreateProgram");
        r.compile = (decltype(r.compile))dlsym(r.lib, "nvrtcCompileProgram");
        r.cubin_size = (decltype(r.cubin_size))dlsym(r.lib, "nvrtcGetCUBINSize");
        r.cubin = (decltype(r.cubin))dlsym(r.lib, "nvrtcGetCUBIN");
        r.log_size = (decltype(r.log_size))dlsym(r.lib, "nvrtcGetProgramLogSize");
        r.log = (decltype(r.log))dlsym(r.lib, "nvrtcGetProgramLog");
        r.destroy = (decltype(r.destroy))dlsym(r.lib, "nvrtcDestroyProgram");
        r.err = (decltype(r.err))dlsym(r.lib, "nvrtcGetErrorString");
        r.ok = r.create && r.compile && r.cubin_size && r.cubin && r.log_size && r.log && r.destroy && r.err;
        return r;
    }();
    return n;
}

// ── driver entry points for loading and launching the compiled module ──
struct Driver {
    CUresult (*module_load)(CUmodule*, const void*) = nullptr;
    CUresult (*module_unload)(CUmodule) = nullptr;
    CUresult (*get_function)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**) = nullptr;
    bool ok = false;
};
template <typename F>
bool entry(const char* name, F& fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return false;
    fn = (F)p;
    return true;
}
Driver& driver() {
    static Driver d = [] {
        Driver r;
        r.ok = entry("cuModuleLoadData", r.module_load) && entry("cuModuleUnload", r.module_unload) &&
               entry("cuModuleGetFunction", r.get_function) && entry("cuLaunchKernel", r.launch);
        return r;
    }();
    return d;
}

// ── code generation ──
struct Gen {
    const sanic_generic_desc* d;
    std::ostringstream out;
    int fresh = 0;
    std::string err;
    std::string inner;      // name of the inner contraction variable while a contracted leaf is rendered, else empty

    std::string tmp() { return "t" + std::to_string(fresh++); }

    static std::string lit(double v) {
        const float f = (float)v;
        uint32_t bits;
        memcpy(&bits, &f, 4);
        char buf[48];
        snprintf(buf, sizeof buf, "__uint_as_float(0x%08xu)", bits);
        return buf;
    }

    // window coordinate j of the flattened stream position `s` (row-major over stream_extent; extents are literals, so the
    // divisions are by constants)
    std::string window_coord(const std::string& s, int j) const {
        long long below = 1;
        for (int i = j + 1; i < d->stream_dims; ++i) below *= d->stream_extent[i];
        std::ostringstream a;
        a << "((" << s << " / " << below << "LL)";
        if (j > 0) a << " % " << (long long)d->stream_extent[j] << "LL";
        a << ")";
        return a.str();
    }

    // element index of operand k at the current point; `s` is the name of the stream variable ("" outside the loop)
    std::string address(int k, const std::string& s) {
        const sanic_operand& o = d->operands[k];
        std::ostringstream a;
        a << "(" << (long long)o.offset << "LL";
        for (int ax = 0; ax < d->n_axes; ++ax)
            if (o.stride[ax] != 0) a << " + c" << ax << " * " << (long long)o.stride[ax] << "LL";
        if (!s.empty() && d->stream_dims > 1) {
            for (int j = 0; j < d->stream_dims; ++j)
                if (o.stream_sub_stride[j] != 0) a << " + " << window_coord(s, j) << " * " << (long long)o.stream_sub_stride[j] << "LL";
        } else if (!s.empty() && o.stream_stride != 0) a << " + " << s << " * " << (long long)o.stream_stride << "LL";
        if (!inner.empty() && o.inner_stride != 0) a << " + " << inner << " * " << (long long)o.inner_stride << "LL";
        a << ")";
        return a.str();
    }

    std::string load(int k, const std::string& s, const std::string& indent) {
        const sanic_operand& o = d->operands[k];
        const std::string t = tmp(), idx = address(k, s), base = "bufs.p[" + std::to_string(o.buffer) + "]";
        switch (o.dtype) {
            case SANIC_F32: out << indent << "const float " << t << " = ((const float*)" << base << ")[" << idx << "];\n"; break;
            case SANIC_BF16: out << indent << "const float " << t << " = widen_bf16(((const unsigned short*)" << base << ")[" << idx << "]);\n"; break;
            case SANIC_U32: out << indent << "const float " << t << " = (float)((const unsigned*)" << base << ")[" << idx << "];\n"; break;
            case SANIC_I4: out << indent << "const float " << t << " = load_i4((const unsigned char*)" << base << ", " << idx << ");\n"; break;
            default: err = "generic emitter: operand dtype not supported"; out << indent << "const float " << t << " = 0.0f;\n";
        }
        return t;
    }

    // Renders one postfix program; returns the name of the value. `s`: stream variable or "".
    std::string program(const sanic_expr& e, const std::string& s, const std::string& indent, const char* item, const char* a,
                        const char* b, const char* f, const char* result) {
        std::vector<std::string> st;
        auto pop = [&]() -> std::string {
            if (st.empty()) { err = "generic emitter: expression stack underflow"; return "0.0f"; }
            std::string v = st.back(); st.pop_back(); return v;
        };
        auto named = [&](const char* base, int i, const char* what) {
            if (!base) { err = std::string("generic emitter: ") + what + " read outside its program"; st.push_back("0.0f"); }
            else st.push_back(std::string(base) + std::to_string(i));
        };
        if (e.first < 0 || e.count < 0 || e.first + e.count > d->n_ops) { err = "generic emitter: program outside the op array"; return "0.0f"; }
        for (int i = e.first; i < e.first + e.count; ++i) {
            const sanic_expr_op& op = d->ops[i];
            auto unary = [&](const char* fn) { std::string x = pop(), t = tmp(); out << indent << "const float " << t << " = " << fn << "(" << x << ");\n"; st.push_back(t); };
            auto binary = [&](const char* l, const char* m, const char* r) {
                std::string y = pop(), x = pop(), t = tmp();
                out << indent << "const float " << t << " = " << l << x << m << y << r << ";\n"; st.push_back(t);
            };
            switch (op.op) {
                case SANIC_X_CONST: st.push_back(lit(op.value)); break;
                case SANIC_X_LOAD:
                    if (op.arg < 0 || op.arg >= d->n_operands) { err = "generic emitter: operand index out of range"; st.push_back("0.0f"); }
                    else st.push_back(load(op.arg, s, indent));
                    break;
                case SANIC_X_GATHER:
                case SANIC_X_GATHER_PAD: {
                    // index = round(value), half away from zero, then a bounds check (src/interp.rs:378-379); an index out
                    // of range reads 0 and leaves code 51 in the status word
                    if (op.arg < 0 || op.arg >= d->n_operands) { err = "generic emitter: operand index out of range"; st.push_back("0.0f"); break; }
                    const sanic_operand& o = d->operands[op.arg];
                    if (o.gather_extent <= 0) { err = "generic emitter: a gathered operand needs a gather extent"; st.push_back("0.0f"); break; }
                    if (o.dtype == SANIC_I4) { err = "generic emitter: gather of an int4 operand is not supported"; st.push_back("0.0f"); break; }
                    const std::string idx = pop(), gi = tmp(), t = tmp();
                    const std::string base = "bufs.p[" + std::to_string(o.buffer) + "]";
                    const std::string at = "[" + address(op.arg, s) + " + " + gi + " * " + std::to_string((long long)o.gather_stride) + "LL]";
                    out << indent << "const long long " << gi << " = (long long)roundf(" << idx << ");\n";
                    out << indent << "float " << t << " = 0.0f;\n";
                    out << indent << "if (" << gi << " >= 0 && " << gi << " < " << (long long)o.gather_extent << "LL) " << t << " = ";
                    if (o.dtype == SANIC_F32) out << "((const float*)" << base << ")" << at;
                    else if (o.dtype == SANIC_BF16) out << "widen_bf16(((const unsigned short*)" << base << ")" << at << ")";
                    else if (o.dtype == SANIC_U32) out << "(float)((const unsigned*)" << base << ")" << at;
                    else err = "generic emitter: operand dtype not supported";
                    if (op.op == SANIC_X_GATHER) out << "; else atomicCAS(status, 0, 51);\n";
                    else out << ";\n";
                    st.push_back(t);
                    break;
                }
                case SANIC_X_COORD:
                    if (op.arg == d->n_axes) {
                        if (s.empty()) { err = "generic emitter: stream coordinate read outside the fold body"; st.push_back("0.0f"); }
                        else st.push_back("(float)" + s);
                    } else if (op.arg == d->n_axes + 1) {
                        if (inner.empty()) { err = "generic emitter: inner coordinate read outside a contracted leaf"; st.push_back("0.0f"); }
                        else st.push_back("(float)" + inner);
                    } else if (op.arg >= d->n_axes + 2 && op.arg < d->n_axes + 2 + d->stream_dims && d->stream_dims > 1) {
                        if (s.empty()) { err = "generic emitter: window coordinate read outside the fold body"; st.push_back("0.0f"); }
                        else st.push_back("(float)" + window_coord(s, op.arg - d->n_axes - 2));
                    } else if (op.arg >= 0 && op.arg < d->n_axes) st.push_back("(float)c" + std::to_string(op.arg));
                    else { err = "generic emitter: coordinate axis out of range"; st.push_back("0.0f"); }
                    break;
                case SANIC_X_ITEM: named(item, op.arg, "Item"); break;
                case SANIC_X_A: named(a, op.arg, "A"); break;
                case SANIC_X_B: named(b, op.arg, "B"); break;
                case SANIC_X_F: named(f, op.arg, "F"); break;
                case SANIC_X_RESULT: if (!result) { err = "generic emitter: Result read outside the epilogue"; st.push_back("0.0f"); } else st.push_back(result); break;
                case SANIC_X_ADD: binary("", " + ", ""); break;
                case SANIC_X_SUB: binary("", " - ", ""); break;
                case SANIC_X_MUL: binary("", " * ", ""); break;
                case SANIC_X_DIV: binary("", " / ", ""); break;
                case SANIC_X_MAX: binary("fmaxf(", ", ", ")"); break;
                case SANIC_X_MIN: binary("fminf(", ", ", ")"); break;
                case SANIC_X_LT: binary("((", " < ", ") ? 1.0f : 0.0f)"); break;
                case SANIC_X_NEG: unary("-"); break;
                case SANIC_X_RECIP: unary("1.0f / "); break;
                case SANIC_X_EXP: unary("expf"); break;
                case SANIC_X_LOG: unary("logf"); break;
                case SANIC_X_SQRT: unary("sqrtf"); break;
                case SANIC_X_TANH: unary("tanhf"); break;
                case SANIC_X_SIN: unary("sinf"); break;
                case SANIC_X_COS: unary("cosf"); break;
                case SANIC_X_WHERE: {
                    std::string bb = pop(), aa = pop(), c = pop(), t = tmp();
                    out << indent << "const float " << t << " = (" << c << " != 0.0f) ? " << aa << " : " << bb << ";\n";
                    st.push_back(t);
                    break;
                }
                case SANIC_X_ROUND:
                    if (op.arg == SANIC_BF16) unary("round_bf16");
                    else if (op.arg != SANIC_F32) err = "generic emitter: RoundTo width not supported";
                    break;
                default: err = "generic emitter: unknown op";
            }
        }
        if (st.size() != 1) { err = "generic emitter: a program must leave exactly one value"; return "0.0f"; }
        return st.back();
    }
};

constexpr const char* PRELUDE = R"(
struct Bufs { const void* p[16]; };
__device__ __forceinline__ float widen_bf16(unsigned short h) { return __uint_as_float(((unsigned)h) << 16); }
__device__ __forceinline__ unsigned short narrow_bf16(float f) {
    unsigned b = __float_as_uint(f);
    if (f != f) return (unsigned short)((b >> 16) | 0x0040u);
    return (unsigned short)((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float round_bf16(float f) { return widen_bf16(narrow_bf16(f)); }
__device__ __forceinline__ float load_i4(const unsigned char* p, long long i) {
    const unsigned byte = p[i >> 1];
    return (float)(int)((i & 1) ? (byte >> 4) : (byte & 15u)) - 8.0f;
}
__device__ __forceinline__ unsigned store_u32(float f) {
    if (!(f > 0.0f)) return 0u;
    if (f >= 4294967296.0f) return 0xFFFFFFFFu;
    return (unsigned)f;
}
)";

int64_t grid_points(const sanic_generic_desc* d) {
    int64_t n = 1;
    for (int a = 0; a < d->n_axes; ++a) n *= d->extent[a];
    return n;
}

int32_t validate(sanic_ctx* ctx, const sanic_generic_desc* d) {
    if (!d) return sanic_fail(ctx, SANIC_ERR_INVALID, "generic emitter: null descriptor");
    SANIC_REQUIRE(ctx, d->n_axes >= 0 && d->n_axes <= SANIC_MAX_AXES, "generic emitter: 0..6 grid axes");
    for (int a = 0; a < d->n_axes; ++a) SANIC_REQUIRE(ctx, d->extent[a] > 0, "generic emitter: grid extents must be positive");
    SANIC_REQUIRE(ctx, d->n_operands >= 0 && d->n_operands <= 64 && (d->n_operands == 0 || d->operands), "generic emitter: bad operand table");
    for (int k = 0; k < d->n_operands; ++k)
        SANIC_REQUIRE(ctx, d->operands[k].buffer >= 0 && d->operands[k].buffer < 16, "generic emitter: buffer index 0..15");
    SANIC_REQUIRE(ctx, d->n_ops >= 0 && (d->n_ops == 0 || d->ops), "generic emitter: bad op array");
    SANIC_REQUIRE(ctx, d->out_dtype == SANIC_F32 || d->out_dtype == SANIC_BF16 || d->out_dtype == SANIC_U32, "generic emitter: bad output dtype");
    SANIC_REQUIRE(ctx, d->stream >= 0, "generic emitter: negative stream extent");
    SANIC_REQUIRE(ctx, d->stream_dims >= 0 && d->stream_dims <= 3, "generic emitter: a streamed window has at most 3 axes");
    if (d->stream_dims > 1) {
        long long prod = 1;
        for (int j = 0; j < d->stream_dims; ++j) {
            SANIC_REQUIRE(ctx, d->stream_extent[j] > 0, "generic emitter: window extents must be positive");
            prod *= d->stream_extent[j];
        }
        SANIC_REQUIRE(ctx, prod == d->stream, "generic emitter: the window's extents must multiply to the streamed extent");
    }
    if (d->stream > 0) {
        SANIC_REQUIRE(ctx, d->n_slots >= 1 && d->n_slots <= SANIC_MAX_SLOTS && d->identity && d->into && d->combine, "generic emitter: 1..8 slots with identity, into and combine");
        SANIC_REQUIRE(ctx, d->n_leaves >= 0 && d->n_leaves <= 16 && (d->n_leaves == 0 || d->leaves), "generic emitter: 0..16 leaves");
        SANIC_REQUIRE(ctx, d->lanes == 1 || d->lanes == 32, "generic emitter: lanes is 1 (one thread per point) or 32 (a warp per point)");
        SANIC_REQUIRE(ctx, !d->lane_axis || (d->lanes == 32 && d->n_axes >= 1 && !d->interleave),
                      "generic emitter: a lane-distributed output axis needs lanes = 32, a grid axis, and no interleave");
        SANIC_REQUIRE(ctx, d->warps >= 0 && d->warps <= 8 && (d->warps <= 1 || d->lanes == 32),
                      "generic emitter: 1..8 warps per point, more than one only with lanes = 32");
    }
    return SANIC_OK;
}

// Does a program read the given grid axis (through a coordinate or through an operand that steps along it)?
bool reads_axis(const sanic_generic_desc* d, const sanic_expr& e, int axis) {
    for (int i = e.first; i < e.first + e.count && i < d->n_ops; ++i) {
        const sanic_expr_op& op = d->ops[i];
        if (op.op == SANIC_X_COORD && op.arg == axis) return true;
        if ((op.op == SANIC_X_LOAD || op.op == SANIC_X_GATHER || op.op == SANIC_X_GATHER_PAD) && op.arg >= 0 && op.arg < d->n_operands &&
            d->operands[op.arg].stride[axis] != 0) return true;
    }
    return false;
}

// The tail every schedule shares: epilogue, conditional store, narrowed store at `index`.
void render_store(Gen& g, const sanic_generic_desc* d, std::string result, const std::string& index) {
    std::ostringstream& o = g.out;
    if (d->epilogue.count > 0) {
        o << "    const float fv = " << result << ";\n";
        result = g.program(d->epilogue, "", "    ", nullptr, nullptr, nullptr, nullptr, "fv");
    }
    if (d->store_if.count > 0) {
        // the in-place form: where(c, x, s) written into s's own buffer stores only where c != 0 and never loads s
        // (src/emit_metal.rs:1118-1178)
        const std::string c = g.program(d->store_if, "", "    ", nullptr, nullptr, nullptr, nullptr, nullptr);
        o << "    if (!(" << c << " != 0.0f)) return;\n";
    }
    switch (d->out_dtype) {
        case SANIC_F32: o << "    ((float*)outp)[" << index << "] = " << result << ";\n"; break;
        case SANIC_BF16: o << "    ((unsigned short*)outp)[" << index << "] = narrow_bf16(" << result << ");\n"; break;
        default: o << "    ((unsigned*)outp)[" << index << "] = store_u32(" << result << ");\n"; break;
    }
    o << "}\n";
}

// Cooperative fold with a lane-distributed output axis (FoldSched::lane_axis, src/plan.rs:434-455): the last grid axis
// is spread over the 32 lanes of a warp, so a warp owns 32 neighbouring output points that share everything not
// spanning that axis. Each lane carries its own accumulator; a contracted leaf that does not read the lane axis (the
// score of an attention fold) is computed ONCE per warp, its inner axis split over the lanes and summed with a
// butterfly, instead of once per output point. With several warps the streamed axis is split over them in contiguous
// chunks and the warp partials merge in warp order through shared memory.
void render_lane_axis(Gen& g, const sanic_generic_desc* d) {
    std::ostringstream& o = g.out;
    const int S = d->n_slots, last = d->n_axes - 1;
    const int W = d->warps > 1 ? d->warps : 1;
    const long long ext = (long long)d->extent[last], passes = (ext + 31) / 32, n = (long long)d->stream;
    long long outer = 1;
    for (int a = 0; a < last; ++a) outer *= d->extent[a];
    const long long units = outer * passes;       // one warp (or one block of W warps) per 32 points of the lane axis
    o << PRELUDE;
    o << "extern \"C\" __global__ void __launch_bounds__(256) sanic_generic(Bufs bufs, void* outp, int* status) {\n";
    o << "    const int lane = threadIdx.x & 31;\n";
    if (W > 1) o << "    const int warp = threadIdx.x >> 5;\n    const long long unit = blockIdx.x;\n";
    else o << "    const long long unit = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;\n";
    o << "    if (unit >= " << units << "LL) return;\n";
    o << "    long long rem = unit / " << passes << "LL;\n";
    o << "    const long long cl = (unit % " << passes << "LL) * 32 + lane;\n";
    o << "    const bool active = cl < " << ext << "LL;\n";
    o << "    const long long c" << last << " = active ? cl : " << (ext - 1) << "LL;   // idle lanes shadow the last point and never store\n";
    o << "    const long long outer = rem;\n";
    for (int a = last - 1; a >= 0; --a)
        o << "    const long long c" << a << " = rem % " << (long long)d->extent[a] << "LL; rem /= " << (long long)d->extent[a] << "LL;\n";
    o << "    (void)rem;\n";
    for (int i = 0; i < S; ++i) o << "    float acc" << i << " = " << Gen::lit(d->identity[i]) << ";\n";
    const long long B = n < W ? n : W;            // chunks of the streamed axis, one per warp
    if (W > 1) {
        o << "    const long long s_lo = (warp < " << B << ") ? (warp * " << n << "LL) / " << B << " : 0;\n";
        o << "    const long long s_hi = (warp < " << B << ") ? ((warp + 1) * " << n << "LL) / " << B << " : 0;\n";
        o << "    #pragma unroll 4\n    for (long long s = s_lo; s < s_hi; ++s) {\n";
    } else {
        o << "    #pragma unroll 4\n    for (long long s = 0; s < " << n << "LL; ++s) {\n";
    }
    const std::string in2 = "        ";
    for (int l = 0; l < d->n_leaves; ++l) {
        const long long R = d->leaf_inner ? (long long)d->leaf_inner[l] : 0;
        if (R > 1) {
            const bool shared = !reads_axis(d, d->leaves[l], last);
            o << in2 << "float x" << l << " = 0.0f;\n";
            if (shared) o << in2 << "for (long long r" << l << " = lane; r" << l << " < " << R << "LL; r" << l << " += 32) {\n";
            else o << in2 << "for (long long r" << l << " = 0; r" << l << " < " << R << "LL; ++r" << l << ") {\n";
            g.inner = "r" + std::to_string(l);
            const std::string v = g.program(d->leaves[l], "s", in2 + "    ", nullptr, nullptr, nullptr, nullptr, nullptr);
            g.inner.clear();
            o << in2 << "    x" << l << " += " << v << ";\n" << in2 << "}\n";
            if (shared) o << in2 << "for (int off = 16; off > 0; off >>= 1) x" << l << " += __shfl_xor_sync(0xffffffffu, x" << l << ", off);\n";
        } else {
            const std::string v = g.program(d->leaves[l], "s", in2, nullptr, nullptr, nullptr, nullptr, nullptr);
            o << in2 << "const float x" << l << " = " << v << ";\n";
        }
    }
    for (int i = 0; i < S; ++i) {
        const std::string v = g.program(d->into[i], "s", in2, "x", nullptr, nullptr, nullptr, nullptr);
        o << in2 << "const float el" << i << " = " << v << ";\n";
    }
    for (int i = 0; i < S; ++i) {
        const std::string v = g.program(d->combine[i], "s", in2, nullptr, "acc", "el", nullptr, nullptr);
        o << in2 << "const float na" << i << " = " << v << ";\n";
    }
    for (int i = 0; i < S; ++i) o << in2 << "acc" << i << " = na" << i << ";\n";
    o << "    }\n";
    if (W > 1) {
        o << "    __shared__ float part[" << W << "][" << S << "][32];\n";
        for (int i = 0; i < S; ++i) o << "    part[warp][" << i << "][lane] = acc" << i << ";\n";
        o << "    __syncthreads();\n    if (warp != 0) return;\n";
        for (int w = 1; w < W && w < B; ++w) {
            o << "    {\n";
            for (int i = 0; i < S; ++i) o << in2 << "const float pw" << i << " = part[" << w << "][" << i << "][lane];\n";
            for (int i = 0; i < S; ++i) {
                const std::string v = g.program(d->combine[i], "", in2, nullptr, "acc", "pw", nullptr, nullptr);
                o << in2 << "const float mw" << i << " = " << v << ";\n";
            }
            for (int i = 0; i < S; ++i) o << in2 << "acc" << i << " = mw" << i << ";\n";
            o << "    }\n";
        }
    }
    o << "    if (!active) return;\n";
    const std::string result = g.program(d->project, "", "    ", nullptr, nullptr, nullptr, "acc", nullptr);
    render_store(g, d, result, "outer * " + std::to_string(ext) + "LL + cl");
}

// The whole kernel as CUDA C text.
int32_t render(sanic_ctx* ctx, const sanic_generic_desc* d, std::string* text) {
    int32_t rc = validate(ctx, d);
    if (rc != SANIC_OK) return rc;
    Gen g{d};
    std::ostringstream& o = g.out;
    if (d->stream > 0 && d->lanes == 32 && d->lane_axis) {
        render_lane_axis(g, d);
        if (!g.err.empty()) return sanic_fail(ctx, SANIC_ERR_INVALID, g.err);
        *text = o.str();
        return SANIC_OK;
    }
    const int64_t points = grid_points(d);
    const bool fold = d->stream > 0;
    const bool coop = fold && d->lanes == 32;
    const int W = (coop && d->warps > 1) ? d->warps : 1;      // warps per output point
    const long long T = 32LL * W;                             // threads per output point
    o << PRELUDE;
    o << "extern \"C\" __global__ void __launch_bounds__(256) sanic_generic(Bufs bufs, void* outp, int* status) {\n";
    if (coop && W > 1) {
        // a block per output point; `lane` numbers its threads across the warps, in chunk order
        o << "    const long long gid = blockIdx.x;\n";
        o << "    const int lane = threadIdx.x;\n";
    } else if (coop) {
        o << "    const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;\n";
        o << "    const int lane = threadIdx.x & 31;\n";
    } else {
        o << "    const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;\n";
    }
    o << "    if (gid >= " << (long long)points << "LL) return;\n";
    // row-major decode of the grid point, last axis fastest (src/codegen.rs grid decode)
    o << "    long long rem = gid;\n";
    for (int a = d->n_axes - 1; a >= 0; --a) {
        o << "    const long long c" << a << " = rem % " << (long long)d->extent[a] << "LL; rem /= " << (long long)d->extent[a] << "LL;\n";
    }
    o << "    (void)rem;\n";
    std::string result;
    if (fold) {
        const int S = d->n_slots;
        for (int i = 0; i < S; ++i) o << "    float acc" << i << " = " << Gen::lit(d->identity[i]) << ";\n";
        const long long n = (long long)d->stream;
        if (coop) {
            const long long B = n < T ? n : T;
            if (d->interleave) {
                o << "    #pragma unroll 4\n    for (long long s = lane; s < " << n << "LL; s += " << T << ") {\n";
            } else {
                o << "    const long long s_lo = (lane < " << B << ") ? (lane * " << n << "LL) / " << B << " : 0;\n";
                o << "    const long long s_hi = (lane < " << B << ") ? ((lane + 1) * " << n << "LL) / " << B << " : 0;\n";
                o << "    #pragma unroll 4\n    for (long long s = s_lo; s < s_hi; ++s) {\n";
            }
        } else {
            o << "    #pragma unroll 4\n    for (long long s = 0; s < " << n << "LL; ++s) {\n";
        }
        const std::string in2 = "        ";
        for (int l = 0; l < d->n_leaves; ++l) {
            const long long R = d->leaf_inner ? (long long)d->leaf_inner[l] : 0;
            if (R > 1) {
                // a leaf that is itself a contraction: sum over the inner axis in the fold body (the in-body QK^T of
                // the online-softmax fold, src/codegen.rs:27-36,328-351), a left fold from 0 in index order
                o << in2 << "float x" << l << " = 0.0f;\n";
                o << in2 << "for (long long r" << l << " = 0; r" << l << " < " << R << "LL; ++r" << l << ") {\n";
                g.inner = "r" + std::to_string(l);
                const std::string v = g.program(d->leaves[l], "s", in2 + "    ", nullptr, nullptr, nullptr, nullptr, nullptr);
                g.inner.clear();
                o << in2 << "    x" << l << " += " << v << ";\n";
                o << in2 << "}\n";
            } else {
                const std::string v = g.program(d->leaves[l], "s", in2, nullptr, nullptr, nullptr, nullptr, nullptr);
                o << in2 << "const float x" << l << " = " << v << ";\n";
            }
        }
        for (int i = 0; i < S; ++i) {
            const std::string v = g.program(d->into[i], "s", in2, "x", nullptr, nullptr, nullptr, nullptr);
            o << in2 << "const float el" << i << " = " << v << ";\n";
        }
        // every new slot is computed from the OLD accumulator before any slot is overwritten
        for (int i = 0; i < S; ++i) {
            const std::string v = g.program(d->combine[i], "s", in2, nullptr, "acc", "el", nullptr, nullptr);
            o << in2 << "const float na" << i << " = " << v << ";\n";
        }
        for (int i = 0; i < S; ++i) o << in2 << "acc" << i << " = na" << i << ";\n";
        o << "    }\n";
        if (coop) {
            // ordered tree over the lanes: the lower lane is the left operand, lanes without a chunk never take part
            const long long B = n < T ? n : T;
            o << "    #pragma unroll\n    for (int off = 1; off < 32; off <<= 1) {\n";
            for (int i = 0; i < S; ++i) o << "        const float pb" << i << " = __shfl_down_sync(0xffffffffu, acc" << i << ", off);\n";
            o << "        const bool take = ((lane & (2 * off - 1)) == 0) && (lane + off < " << B << ");\n";
            const std::string in2b = "        ";
            for (int i = 0; i < S; ++i) {
                const std::string v = g.program(d->combine[i], "", in2b, nullptr, "acc", "pb", nullptr, nullptr);
                o << in2b << "const float ma" << i << " = " << v << ";\n";
            }
            for (int i = 0; i < S; ++i) o << in2b << "if (take) acc" << i << " = ma" << i << ";\n";
            o << "    }\n";
            if (W > 1) {
                // warp partials meet in shared memory and merge left to right in warp order (the threadgroup-memory
                // merge rounds of the reference's cooperative fold)
                o << "    __shared__ float part[" << W << "][" << S << "];\n";
                o << "    if ((lane & 31) == 0) {";
                for (int i = 0; i < S; ++i) o << " part[lane >> 5][" << i << "] = acc" << i << ";";
                o << " }\n    __syncthreads();\n";
                o << "    if (lane != 0) return;\n";
                for (int w = 1; w < W; ++w) {
                    if (32LL * w >= B) break;      // that warp and the ones after it had no chunk
                    o << "    {\n";
                    const std::string in3 = "        ";
                    for (int i = 0; i < S; ++i) o << in3 << "const float pw" << i << " = part[" << w << "][" << i << "];\n";
                    for (int i = 0; i < S; ++i) {
                        const std::string v = g.program(d->combine[i], "", in3, nullptr, "acc", "pw", nullptr, nullptr);
                        o << in3 << "const float mw" << i << " = " << v << ";\n";
                    }
                    for (int i = 0; i < S; ++i) o << in3 << "acc" << i << " = mw" << i << ";\n";
                    o << "    }\n";
                }
            } else {
                o << "    if (lane != 0) return;\n";
            }
        }
        result = g.program(d->project, "", "    ", nullptr, nullptr, nullptr, "acc", nullptr);
    } else {
        result = g.program(d->project, "", "    ", nullptr, nullptr, nullptr, nullptr, nullptr);
    }
    render_store(g, d, result, "gid");
    if (!g.err.empty()) return sanic_fail(ctx, SANIC_ERR_INVALID, g.err);
    *text = o.str();
    return SANIC_OK;
}

// Kernel dedup across isomorphic stages (src/emit_metal.rs:1281-1330 canonicalises each kernel's source and keeps one entry
// point per body): here buffers bind positionally at launch and every extent and dtype is baked into the text, so two
// stages that differ only in their buffers render the SAME text, and the text is the key. One compilation per text per
// process; every kernel object still loads its own module (a module belongs to a context).
struct CubinCache {
    std::mutex mu;
    std::map<std::string, std::vector<char>> by_text;
    long long compiled = 0, reused = 0;
};
CubinCache& cubin_cache() { static CubinCache c; return c; }

int32_t compile_cubin(sanic_ctx* ctx, const std::string& text, std::vector<char>* cubin) {
    {
        CubinCache& c = cubin_cache();
        std::lock_guard<std::mutex> lock(c.mu);
        auto it = c.by_text.find(text);
        if (it != c.by_text.end()) { *cubin = it->second; ++c.reused; return SANIC_OK; }
    }
    Nvrtc& n = nvrtc();
    if (!n.ok) return sanic_fail(ctx, SANIC_ERR_UNSUPPORTED, "generic emitter: the NVRTC library could not be loaded");
    nvrtcProgram prog;
    nvrtcResult r = n.create(&prog, text.c_str(), "sanic_generic.cu", 0, nullptr, nullptr);
    if (r != NVRTC_SUCCESS) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("nvrtcCreateProgram: ") + n.err(r));
    const char* opts[] = {"--gpu-architecture=sm_100a", "-lineinfo", "--fmad=true"};
    r = n.compile(prog, 3, opts);
    if (r != NVRTC_SUCCESS) {
        size_t ls = 0;
        n.log_size(prog, &ls);
        std::string log(ls, '\0');
        if (ls) n.log(prog, &log[0]);
        n.destroy(&prog);
        return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("generated kernel failed to compile: ") + n.err(r) + "\n" + log);
    }
    size_t sz = 0;
    n.cubin_size(prog, &sz);
    cubin->resize(sz);
    if (sz) n.cubin(prog, cubin->data());
    n.destroy(&prog);
    if (!sz) return sanic_fail(ctx, SANIC_ERR_CUDA, "generated kernel: empty cubin");
    CubinCache& c = cubin_cache();
    std::lock_guard<std::mutex> lock(c.mu);
    ++c.compiled;
    if (c.by_text.size() < 4096) c.by_text.emplace(text, *cubin);
    return SANIC_OK;
}

// A descriptive name (kind, grid, streamed extent, schedule), as the reference composes one per kernel
// (kernel_name, src/emit_metal.rs:1340-1370): what a stage listing or a profile shows instead of one entry-point name.
std::string describe(const sanic_generic_desc* d) {
    std::ostringstream o;
    if (d->stream > 0) o << "fold" << d->n_slots; else o << "map";
    o << "_g";
    for (int a = 0; a < d->n_axes; ++a) o << (a ? "x" : "") << (long long)d->extent[a];
    if (d->n_axes == 0) o << "1";
    if (d->stream > 0) {
        o << "_s";
        if (d->stream_dims > 1) for (int j = 0; j < d->stream_dims; ++j) o << (j ? "x" : "") << (long long)d->stream_extent[j];
        else o << (long long)d->stream;
        if (d->lanes == 32) o << (d->lane_axis ? "_laneaxis" : (d->interleave ? "_lanes_interleaved" : "_lanes")) << (d->warps > 1 ? "_w" + std::to_string(d->warps) : "");
        else o << "_thread";
    }
    o << (d->out_dtype == SANIC_BF16 ? "_bf16" : (d->out_dtype == SANIC_U32 ? "_u32" : "_f32"));
    return o.str();
}

}  // namespace

struct sanic_generic_kernel {
    std::string name;
    CUmodule module = nullptr;
    CUfunction fn = nullptr;
    int64_t points = 0;     // launch units
    int lanes = 1;          // threads per launch unit
    int block = 256;
    int n_buffers = 0;
};

extern "C" {

int32_t sanic_generic_source(sanic_ctx* ctx, const sanic_generic_desc* d, char* buf, size_t cap, size_t* needed) {
    std::string text;
    int32_t rc = render(ctx, d, &text);
    if (rc != SANIC_OK) return rc;
    if (needed) *needed = text.size() + 1;
    if (buf && cap) {
        const size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
        memcpy(buf, text.data(), n);
        buf[n] = '\0';
    }
    return SANIC_OK;
}

int32_t sanic_generic_cubin_size(sanic_ctx* ctx, const sanic_generic_desc* d, size_t* bytes) {
    std::string text;
    int32_t rc = render(ctx, d, &text);
    if (rc != SANIC_OK) return rc;
    std::vector<char> cubin;
    rc = compile_cubin(ctx, text, &cubin);
    if (rc != SANIC_OK) return rc;
    if (bytes) *bytes = cubin.size();
    return SANIC_OK;
}

int32_t sanic_generic_compile(sanic_ctx* ctx, const sanic_generic_desc* d, sanic_generic_kernel** out) {
    if (!ctx || !out) return SANIC_ERR_INVALID;
    *out = nullptr;
    std::string text;
    int32_t rc = render(ctx, d, &text);
    if (rc != SANIC_OK) return rc;
    std::vector<char> cubin;
    rc = compile_cubin(ctx, text, &cubin);
    if (rc != SANIC_OK) return rc;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaFree(nullptr));   // the primary context exists and is current
    Driver& dr = driver();
    if (!dr.ok) return sanic_fail(ctx, SANIC_ERR_CUDA, "generic emitter: driver entry points for module loading not found");
    sanic_generic_kernel* k = new sanic_generic_kernel();
    CUresult cr = dr.module_load(&k->module, cubin.data());
    if (cr != CUDA_SUCCESS) { delete k; return sanic_fail(ctx, SANIC_ERR_CUDA, "cuModuleLoadData failed with code " + std::to_string((int)cr)); }
    cr = dr.get_function(&k->fn, k->module, "sanic_generic");
    if (cr != CUDA_SUCCESS) { dr.module_unload(k->module); delete k; return sanic_fail(ctx, SANIC_ERR_CUDA, "cuModuleGetFunction failed with code " + std::to_string((int)cr)); }
    k->name = describe(d);
    k->points = grid_points(d);
    if (d->stream > 0 && d->lanes == 32 && d->lane_axis) {      // a unit = 32 points of the last axis
        const int64_t ext = d->extent[d->n_axes - 1];
        k->points = k->points / ext * ((ext + 31) / 32);
    }
    k->lanes = (d->stream > 0 && d->lanes == 32) ? 32 * (d->warps > 1 ? d->warps : 1) : 1;
    k->block = k->lanes > 32 ? k->lanes : 256;      // several warps per point: one block per point
    for (int i = 0; i < d->n_operands; ++i) if (d->operands[i].buffer + 1 > k->n_buffers) k->n_buffers = d->operands[i].buffer + 1;
    *out = k;
    return SANIC_OK;
}

int32_t sanic_generic_launch(sanic_ctx* ctx, sanic_generic_kernel* k, const void* const* buffers, int32_t n_buffers, void* out,
                             void* stream) {
    if (!ctx || !k) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, out, "generic launch: null output");
    SANIC_REQUIRE(ctx, n_buffers >= k->n_buffers && n_buffers <= 16, "generic launch: the kernel reads more buffers than were bound");
    struct { const void* p[16]; } bufs = {};
    for (int i = 0; i < n_buffers; ++i) {
        SANIC_REQUIRE(ctx, buffers && (buffers[i] || i >= k->n_buffers), "generic launch: unbound buffer");
        bufs.p[i] = buffers[i];
    }
    const int64_t threads = k->points * k->lanes;
    const int64_t blocks = (threads + k->block - 1) / k->block;
    SANIC_REQUIRE(ctx, blocks <= 0x7FFFFFFFLL, "generic launch: grid too large");
    int* status = ctx->status_dev;
    void* args[] = {&bufs, &out, &status};
    sanic_set_device(ctx);
    CUresult cr = driver().launch(k->fn, (unsigned)blocks, 1, 1, (unsigned)k->block, 1, 1, 0, (CUstream)stream, args, nullptr);
    if (cr != CUDA_SUCCESS) return sanic_fail(ctx, SANIC_ERR_CUDA, "cuLaunchKernel failed with code " + std::to_string((int)cr));
    return SANIC_OK;
}

const char* sanic_generic_kernel_name(sanic_generic_kernel* k) { return k ? k->name.c_str() : ""; }

int32_t sanic_generic_cache_stats(int64_t* compiled, int64_t* reused) {
    CubinCache& c = cubin_cache();
    std::lock_guard<std::mutex> lock(c.mu);
    if (compiled) *compiled = c.compiled;
    if (reused) *reused = c.reused;
    return SANIC_OK;
}

int32_t sanic_generic_destroy(sanic_generic_kernel* k) {
    if (!k) return SANIC_ERR_INVALID;
    if (k->module && driver().ok) driver().module_unload(k->module);
    delete k;
    return SANIC_OK;
}

}  // extern "C"
