// sanic_oracle — CPU restatement of the reference's dense f64 interpreter.
//
// TEST INFRASTRUCTURE ONLY. This file is the parity checker and the timed CPU
// baseline. Nothing in the shipped library links, loads or calls it.
//
// What it restates (paths are relative to the reference project):
//   * src/interp.rs:270-430   eval: every intermediate dense in f64, Reduce is a
//                             left fold from the monoid identity in index order,
//                             Map broadcasting is right-aligned with extent-1
//                             dimensions reading index 0, padded Reindex reads 0.0.
//   * src/interp.rs:472-518   apply_map / monoid_combine scalar semantics.
//   * src/interp.rs:555-643   run_carrier_split: contiguous chunks
//                             [b*n/B, (b+1)*n/B), merge from the first partial,
//                             project once.
//   * src/scalar.rs:120-177   round_to (bf16 RNE on the high half with quiet NaN,
//                             f16 with the same double rounding, f32).
//   * src/ir.rs:1171-1223     matmul = Reduce(Add, Map(Mul, a[...,m,k,1], b[...,1,k,n])).
//   * src/ir.rs:1277-1284     softmax = exp(x - max) / sum.
//   * src/ir.rs:1415-1433     argmax = Min(where(x < max, +inf, coordinate)).
//   * src/ir.rs:1500-1526     silu, causal_mask_like (-1e30).
//   * src/nn.rs:27-151        scaled_dot_product_attention, GQA repeat-interleave.
//   * src/nn.rs:165-212       rms_norm, rope (rotate-half), rope_inv_freq, update_cache.
//   * src/derive.rs:1688-1747 assemble: the combine of Plain / ExpShifted /
//                             AtExtremum slots, including the -inf guard.
//   * examples/llama3_2.rs:95-253  llama3_inv_freq and the decode-step graph.
//   * tests/oracle.rs:49-59   xorshift64* test PRNG.
//   * tests/movement.rs:294-345 sliding-window attention as a padded window reindex.
//
// Parity status: PINNED. tests/test_oracle_pins.py checks this file against the
// literal known answers and seeded self-consistency laws of the reference's own
// tests (tests/nn.rs, tests/compile.rs, tests/group.rs, tests/oracle.rs,
// tests/decode.rs, tests/movement.rs, tests/metal.rs).
//
// One deliberate difference, which changes no value: a matmul does not
// materialise the [.., m, k, n] product tensor before reducing it; it forms each
// product and adds it in the same index order, so every rounding is identical.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr double NEG_INF = -std::numeric_limits<double>::infinity();
constexpr double POS_INF = std::numeric_limits<double>::infinity();

// ───────────────────────── scalar semantics ─────────────────────────
// src/scalar.rs:120-177
inline float bits_f32(uint32_t b) { float f; std::memcpy(&f, &b, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t b; std::memcpy(&b, &f, 4); return b; }

inline uint16_t bf16_bits_of(double v) {
    float f = (float)v;
    uint32_t b = f32_bits(f);
    if (std::isnan(f)) return (uint16_t)((b >> 16) | 0x0040);
    uint32_t r = (b + 0x7FFFu + ((b >> 16) & 1u)) >> 16;
    return (uint16_t)r;
}
inline double bf16_widen(uint16_t h) { return (double)bits_f32(((uint32_t)h) << 16); }
inline double round_bf16(double v) { return bf16_widen(bf16_bits_of(v)); }

inline float half_round(float v) {
    if (std::isnan(v)) return v;
    uint32_t bits = f32_bits(v);
    uint32_t sign = bits >> 31;
    float magnitude = bits_f32(bits & 0x7FFFFFFFu);
    uint32_t mb = f32_bits(magnitude);
    float rounded;
    if (mb >= 0x47800000u) {
        rounded = std::numeric_limits<float>::infinity();
    } else if (mb < 0x38800000u) {
        float ulp = bits_f32(0x33800000u);  // 2^-24
        float n = std::nearbyintf(magnitude / ulp);  // ties to even under the default mode
        rounded = n * ulp;
    } else {
        uint32_t r = (mb + 0xFFFu + ((mb >> 13) & 1u)) & ~0x1FFFu;
        rounded = bits_f32(r);
    }
    return sign ? -rounded : rounded;
}

enum Dtype { DT_F64 = 0, DT_F32 = 1, DT_F16 = 2, DT_BF16 = 3 };
inline double round_to(int dtype, double v) {
    switch (dtype) {
        case DT_F32: return (double)(float)v;
        case DT_F16: return (double)half_round((float)v);
        case DT_BF16: return round_bf16(v);
        default: return v;
    }
}

// src/interp.rs:499-518 (the monoids used on this path)
inline double cmax(double a, double b) { return std::fmax(a, b); }  // f64::max ignores a NaN side, as fmax does
inline double cmin(double a, double b) { return std::fmin(a, b); }

// ───────────────────────── dense tensors ─────────────────────────
struct Value {
    std::vector<size_t> shape;
    std::vector<double> data;
    size_t rank() const { return shape.size(); }
    size_t volume() const { size_t v = 1; for (size_t s : shape) v *= s; return v; }
};

Value make(std::vector<size_t> shape) {
    Value v; v.shape = std::move(shape); v.data.assign(v.volume(), 0.0); return v;
}
Value from_ptr(std::vector<size_t> shape, const double* p) {
    Value v; v.shape = std::move(shape); size_t n = v.volume(); v.data.assign(p, p + n); return v;
}

// Right-aligned broadcasting of a binary map (src/interp.rs:322-347).
template <class F>
Value map2(const Value& a, const Value& b, F f) {
    size_t r = std::max(a.rank(), b.rank());
    std::vector<size_t> sa(r, 1), sb(r, 1), so(r, 1);
    for (size_t i = 0; i < a.rank(); ++i) sa[r - a.rank() + i] = a.shape[i];
    for (size_t i = 0; i < b.rank(); ++i) sb[r - b.rank() + i] = b.shape[i];
    for (size_t i = 0; i < r; ++i) so[i] = std::max(sa[i], sb[i]);
    Value o = make(so);
    std::vector<size_t> stra(r, 0), strb(r, 0);
    size_t acc = 1;
    for (size_t i = r; i-- > 0;) { stra[i] = (sa[i] == 1) ? 0 : acc; acc *= sa[i]; }
    acc = 1;
    for (size_t i = r; i-- > 0;) { strb[i] = (sb[i] == 1) ? 0 : acc; acc *= sb[i]; }
    size_t n = o.volume();
    std::vector<size_t> idx(r, 0);
    size_t ia = 0, ib = 0;
    for (size_t lin = 0; lin < n; ++lin) {
        o.data[lin] = f(a.data[ia], b.data[ib]);
        for (size_t d = r; d-- > 0;) {
            idx[d]++; ia += stra[d]; ib += strb[d];
            if (idx[d] < so[d]) break;
            ia -= stra[d] * so[d]; ib -= strb[d] * so[d]; idx[d] = 0;
        }
    }
    return o;
}
template <class F>
Value map1(const Value& a, F f) {
    Value o = a;
    for (double& x : o.data) x = f(x);
    return o;
}
Value scalar(double v) { Value s; s.data = {v}; return s; }

// Reduce one dimension with a left fold from the identity (src/interp.rs:350-365).
template <class F>
Value reduce(const Value& s, size_t dim, double identity, F combine) {
    std::vector<size_t> oshape;
    for (size_t i = 0; i < s.rank(); ++i) if (i != dim) oshape.push_back(s.shape[i]);
    Value o = make(oshape);
    size_t inner = 1, n = s.shape[dim];
    for (size_t i = dim + 1; i < s.rank(); ++i) inner *= s.shape[i];
    size_t outer = s.volume() / (inner * n);
    for (size_t a = 0; a < outer; ++a)
        for (size_t c = 0; c < inner; ++c) {
            double acc = identity;
            for (size_t i = 0; i < n; ++i) acc = combine(acc, s.data[(a * n + i) * inner + c]);
            o.data[a * inner + c] = acc;
        }
    return o;
}
Value unsqueeze(const Value& s, size_t dim) {
    Value o = s; o.shape.insert(o.shape.begin() + dim, 1); return o;
}
Value transpose_last2(const Value& s) {
    size_t r = s.rank(); size_t m = s.shape[r - 2], n = s.shape[r - 1];
    Value o = s; std::swap(o.shape[r - 2], o.shape[r - 1]);
    size_t batch = s.volume() / (m * n);
    for (size_t b = 0; b < batch; ++b)
        for (size_t i = 0; i < m; ++i)
            for (size_t j = 0; j < n; ++j) o.data[(b * n + j) * m + i] = s.data[(b * m + i) * n + j];
    return o;
}

// matmul over [..., m, k] x [..., k, n] with equal leading dims (src/ir.rs:1171-1223).
Value matmul(const Value& a, const Value& b) {
    size_t ra = a.rank(), rb = b.rank();
    size_t m = a.shape[ra - 2], k = a.shape[ra - 1], n = b.shape[rb - 1];
    size_t batch = a.volume() / (m * k);
    std::vector<size_t> oshape(a.shape.begin(), a.shape.end() - 2);
    oshape.push_back(m); oshape.push_back(n);
    Value o = make(oshape);
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t i = 0; i < m; ++i) {
            const double* ar = &a.data[(bi * m + i) * k];
            const double* bb = &b.data[bi * k * n];
            double* orow = &o.data[(bi * m + i) * n];
            // every output starts at the Add identity and takes its k terms in index order;
            // the k loop is outermost only so that the inner loop walks memory contiguously
            for (size_t j = 0; j < n; ++j) orow[j] = 0.0;
            for (size_t kk = 0; kk < k; ++kk) {
                const double a_ik = ar[kk];
                const double* brow = bb + kk * n;
                for (size_t j = 0; j < n; ++j) orow[j] = orow[j] + a_ik * brow[j];
            }
        }
    return o;
}

// softmax over the last dimension (src/ir.rs:1277-1284).
Value softmax_last(const Value& x) {
    size_t r = x.rank();
    Value mx = reduce(x, r - 1, NEG_INF, cmax);
    Value ex = map1(map2(x, unsqueeze(mx, r - 1), [](double a, double b) { return a - b; }),
                    [](double a) { return std::exp(a); });
    Value nz = reduce(ex, r - 1, 0.0, [](double a, double b) { return a + b; });
    return map2(ex, unsqueeze(nz, r - 1), [](double a, double b) { return a / b; });
}

// GQA: q head h reads kv head h / repeats (src/nn.rs:107-151: the expanded
// [.., kv, repeat, ..] dims are flattened with kv most significant).
Value repeat_interleave_heads(const Value& src, size_t target_heads) {
    size_t r = src.rank(); size_t hd = r - 3;
    size_t h = src.shape[hd], rep = target_heads / h;
    if (rep == 1) return src;
    std::vector<size_t> oshape = src.shape; oshape[hd] = target_heads;
    Value o = make(oshape);
    size_t inner = src.shape[r - 2] * src.shape[r - 1];
    size_t outer = src.volume() / (h * inner);
    for (size_t a = 0; a < outer; ++a)
        for (size_t t = 0; t < target_heads; ++t)
            std::memcpy(&o.data[(a * target_heads + t) * inner], &src.data[(a * h + t / rep) * inner],
                        inner * sizeof(double));
    return o;
}

// scaled_dot_product_attention (src/nn.rs:27-105). q [N,Hq,L,E], k [N,H,S,E], v [N,H,S,Ev].
Value sdpa(const Value& q, Value k, Value v, const Value* mask, bool is_causal, double scale, bool gqa) {
    if (gqa) { k = repeat_interleave_heads(k, q.shape[q.rank() - 3]); v = repeat_interleave_heads(v, q.shape[q.rank() - 3]); }
    Value kt = transpose_last2(k);
    Value scores = map2(matmul(q, kt), scalar(scale), [](double a, double b) { return a * b; });
    size_t r = scores.rank(); size_t L = scores.shape[r - 2], S = scores.shape[r - 1];
    if (is_causal) {
        // causal_mask_like: where(coord(query) < coord(key), -1e30, 0)  (src/ir.rs:1511-1526)
        Value m = make({L, S});
        for (size_t i = 0; i < L; ++i) for (size_t j = 0; j < S; ++j) m.data[i * S + j] = (i < j) ? -1e30 : 0.0;
        scores = map2(scores, m, [](double a, double b) { return a + b; });
    } else if (mask) {
        scores = map2(scores, *mask, [](double a, double b) { return a + b; });
    }
    return matmul(softmax_last(scores), v);
}

// ───────────────────────── carriers (src/derive.rs) ─────────────────────────
enum SlotKindTag { PLAIN_ADD, PLAIN_MAX, PLAIN_MIN, EXP_SHIFTED, AT_EXTREMUM_MAX_TIES_MIN };
struct Slot { SlotKindTag kind; int ref; };  // ref: max_slot for EXP_SHIFTED, key_slot for AT_EXTREMUM

// combine, slot by slot, as assemble() builds it (src/derive.rs:1688-1735).
void carrier_merge(const std::vector<Slot>& slots, const double* a, const double* b, double* out) {
    for (size_t i = 0; i < slots.size(); ++i) {
        const Slot& s = slots[i];
        switch (s.kind) {
            case PLAIN_ADD: out[i] = a[i] + b[i]; break;
            case PLAIN_MAX: out[i] = cmax(a[i], b[i]); break;
            case PLAIN_MIN: out[i] = cmin(a[i], b[i]); break;
            case EXP_SHIFTED: {
                double big = cmax(a[s.ref], b[s.ref]);
                double ra = (NEG_INF < a[s.ref]) ? std::exp(a[s.ref] - big) : 0.0;
                double rb = (NEG_INF < b[s.ref]) ? std::exp(b[s.ref] - big) : 0.0;
                out[i] = a[i] * ra + b[i] * rb;
                break;
            }
            case AT_EXTREMUM_MAX_TIES_MIN: {
                double ka = a[s.ref], kb = b[s.ref];
                out[i] = (ka < kb) ? b[i] : ((kb < ka) ? a[i] : cmin(a[i], b[i]));
                break;
            }
        }
    }
}
void carrier_identity(const std::vector<Slot>& slots, double* out) {
    for (size_t i = 0; i < slots.size(); ++i) {
        switch (slots[i].kind) {
            case PLAIN_ADD: out[i] = 0.0; break;
            case PLAIN_MAX: out[i] = NEG_INF; break;
            case PLAIN_MIN: out[i] = POS_INF; break;
            case EXP_SHIFTED: out[i] = 0.0; break;
            case AT_EXTREMUM_MAX_TIES_MIN: out[i] = POS_INF; break;
        }
    }
}

// Stage 1 + stage 2 of run_carrier_split for one grid point (src/interp.rs:597-640).
// lift(i, el) fills the element's accumulator-shaped value.
template <class Lift>
void fold_split(const std::vector<Slot>& slots, size_t n, size_t blocks, Lift lift, double* acc_out) {
    size_t w = slots.size();
    std::vector<double> partials(blocks * w), el(w), tmp(w);
    for (size_t b = 0; b < blocks; ++b) {
        double* acc = &partials[b * w];
        carrier_identity(slots, acc);
        size_t lo = b * n / blocks, hi = (b + 1) * n / blocks;
        for (size_t i = lo; i < hi; ++i) {
            lift(i, el.data());
            carrier_merge(slots, acc, el.data(), tmp.data());
            std::copy(tmp.begin(), tmp.end(), acc);
        }
    }
    std::copy(partials.begin(), partials.begin() + w, acc_out);
    for (size_t b = 1; b < blocks; ++b) {
        carrier_merge(slots, acc_out, &partials[b * w], tmp.data());
        std::copy(tmp.begin(), tmp.end(), acc_out);
    }
}

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// tests/oracle.rs:49-59 — xorshift64* mapped to [-1, 1).
void orc_xorshift_uniform(uint64_t* state, double* out, size_t n) {
    uint64_t x = *state;
    for (size_t i = 0; i < n; ++i) {
        x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
        out[i] = ((double)((x * 0x2545F4914F6CDD1DULL) >> 11) / (double)(1ULL << 53)) * 2.0 - 1.0;
    }
    *state = x;
}

// Box-Muller over the same xorshift64* stream: the seeded N(0,1) source for
// synthetic workloads (two uniforms per pair of normals).
void orc_xorshift_normal(uint64_t* state, double* out, size_t n) {
    uint64_t x = *state;
    auto next01 = [&]() {
        x ^= x >> 12; x ^= x << 25; x ^= x >> 27;
        return ((double)((x * 0x2545F4914F6CDD1DULL) >> 11) + 0.5) / (double)(1ULL << 53);
    };
    for (size_t i = 0; i < n; i += 2) {
        double u1 = next01(), u2 = next01();
        double r = std::sqrt(-2.0 * std::log(u1)), t = 6.283185307179586476925 * u2;
        out[i] = r * std::cos(t);
        if (i + 1 < n) out[i + 1] = r * std::sin(t);
    }
    *state = x;
}

void orc_round_to(int dtype, const double* in, double* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = round_to(dtype, in[i]);
}
void orc_to_bf16_bits(const double* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_bits_of(in[i]);
}
void orc_from_bf16_bits(const uint16_t* in, double* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = bf16_widen(in[i]);
}

// int4 storage: unsigned nibble q+8, low nibble = even element
// (src/emit_metal.rs:119-122,179-181; tests/metal.rs:1186-1193).
void orc_w4_pack(const int8_t* q, size_t n, uint8_t* packed) {
    std::memset(packed, 0, (n + 1) / 2);
    for (size_t i = 0; i < n; ++i) packed[i / 2] |= (uint8_t)(((uint8_t)(q[i] + 8)) << ((i & 1) * 4));
}
void orc_w4_unpack(const uint8_t* packed, size_t n, double* out) {
    for (size_t i = 0; i < n; ++i) out[i] = (double)(int)((packed[i / 2] >> ((i & 1) * 4)) & 0xF) - 8.0;
}

// eval(scaled_dot_product_attention). mask (optional) is additive with a 4-d
// shape whose 1-extents broadcast. Returns 0.
int orc_sdpa(const double* q, const double* k, const double* v, const double* mask, const size_t* mask_shape,
             size_t N, size_t Hq, size_t H, size_t L, size_t S, size_t E, size_t Ev, int is_causal, double scale,
             int enable_gqa, double* out) {
    Value Q = from_ptr({N, Hq, L, E}, q), K = from_ptr({N, H, S, E}, k), V = from_ptr({N, H, S, Ev}, v);
    Value M;
    if (mask) M = from_ptr({mask_shape[0], mask_shape[1], mask_shape[2], mask_shape[3]}, mask);
    Value o = sdpa(Q, K, V, mask ? &M : nullptr, is_causal != 0, scale, enable_gqa != 0);
    std::copy(o.data.begin(), o.data.end(), out);
    return 0;
}

// Sliding-window attention in the reference's formulation (tests/movement.rs:294-345):
// K and V are read through a padded window reindex t = s + j - (w-1), j in [0, w);
// out-of-range reads are 0.0 and positions with s + j < w-1 get -1e30 added.
// Query s therefore attends to keys s-w+1 .. s. Scores are scaled before the mask.
int orc_sdpa_window(const double* q, const double* k, const double* v, size_t N, size_t Hq, size_t H, size_t L,
                    size_t E, size_t Ev, size_t window, double scale, double* out) {
    size_t rep = Hq / H;
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t n = 0; n < N; ++n)
        for (size_t h = 0; h < Hq; ++h) {
            const double* Q = q + ((n * Hq + h) * L) * E;
            const double* K = k + ((n * H + h / rep) * L) * E;
            const double* V = v + ((n * H + h / rep) * L) * Ev;
            std::vector<double> sc(window), ex(window);
            for (size_t s = 0; s < L; ++s) {
                for (size_t j = 0; j < window; ++j) {
                    long t = (long)s + (long)j - (long)(window - 1);
                    double acc = 0.0;
                    for (size_t d = 0; d < E; ++d) {
                        double kv = (t < 0 || t >= (long)L) ? 0.0 : K[(size_t)t * E + d];
                        acc = acc + Q[s * E + d] * kv;
                    }
                    acc = acc * scale;
                    sc[j] = acc + ((double)(s + j) < (double)(window - 1) ? -1e30 : 0.0);
                }
                double m = NEG_INF;
                for (size_t j = 0; j < window; ++j) m = cmax(m, sc[j]);
                double z = 0.0;
                for (size_t j = 0; j < window; ++j) { ex[j] = std::exp(sc[j] - m); z = z + ex[j]; }
                for (size_t e = 0; e < Ev; ++e) {
                    double acc = 0.0;
                    for (size_t j = 0; j < window; ++j) {
                        long t = (long)s + (long)j - (long)(window - 1);
                        double vv = (t < 0 || t >= (long)L) ? 0.0 : V[(size_t)t * Ev + e];
                        acc = acc + (ex[j] / z) * vv;
                    }
                    out[((n * Hq + h) * L + s) * Ev + e] = acc;
                }
            }
        }
    return 0;
}

// run_carrier_split of the derived online-softmax carrier (m, l, o):
// slots (Plain(Max), ExpShifted{0}, ExpShifted{0}), into = (score, 1, v),
// project = o / l (tests/laws.rs:107-126). One grid point per (n, h, l, e), so
// the (m, l) slots are recomputed per value feature exactly as the interpreter
// does. The scores leaf is the in-body contraction scale*QK^T (+ mask).
// carriers_out (optional) receives the merged raw accumulators [N,Hq,L,2+Ev].
int orc_sdpa_carrier_split(const double* q, const double* k, const double* v, const double* mask,
                           const size_t* mask_shape, size_t N, size_t Hq, size_t H, size_t L, size_t S, size_t E,
                           size_t Ev, int is_causal, double scale, int enable_gqa, size_t blocks, double* out,
                           double* carriers_out) {
    if (blocks < 1 || blocks > S) return 1;  // src/interp.rs:570-574
    size_t rep = enable_gqa ? Hq / H : 1;
    std::vector<Slot> slots = {{PLAIN_MAX, 0}, {EXP_SHIFTED, 0}, {EXP_SHIFTED, 0}};
#pragma omp parallel for collapse(2) schedule(static)
    for (size_t n = 0; n < N; ++n)
        for (size_t h = 0; h < Hq; ++h) {
            size_t hk = h / rep;
            std::vector<double> score(S);
            for (size_t l = 0; l < L; ++l) {
                const double* Q = q + ((n * Hq + h) * L + l) * E;
                for (size_t s = 0; s < S; ++s) {
                    const double* K = k + ((n * H + hk) * S + s) * E;
                    double acc = 0.0;
                    for (size_t d = 0; d < E; ++d) acc = acc + Q[d] * K[d];
                    acc = acc * scale;
                    if (is_causal) acc = acc + ((l < s) ? -1e30 : 0.0);
                    else if (mask) {
                        size_t mi = ((((mask_shape[0] == 1 ? 0 : n) * mask_shape[1] + (mask_shape[1] == 1 ? 0 : h)) *
                                      mask_shape[2] + (mask_shape[2] == 1 ? 0 : l)) * mask_shape[3] +
                                     (mask_shape[3] == 1 ? 0 : s));
                        acc = acc + mask[mi];
                    }
                    score[s] = acc;
                }
                for (size_t e = 0; e < Ev; ++e) {
                    const double* V = v + ((n * H + hk) * S) * Ev + e;
                    double acc[3] = {0.0, 0.0, 0.0};
                    fold_split(slots, S, blocks,
                               [&](size_t i, double* el) { el[0] = score[i]; el[1] = 1.0; el[2] = V[i * Ev]; }, acc);
                    out[((n * Hq + h) * L + l) * Ev + e] = acc[2] / acc[1];
                    if (carriers_out) {
                        double* c = carriers_out + ((n * Hq + h) * L + l) * (2 + Ev);
                        c[0] = acc[0]; c[1] = acc[1]; c[2 + e] = acc[2];
                    }
                }
            }
        }
    return 0;
}

// Stage-2 merge of per-shard (m, l, o) carriers, then project: what the
// cross-device merge must reproduce (src/interp.rs:632-639).
// parts: [n_parts, rows, 2+Ev]; out: [rows, Ev].
void orc_carrier_merge_mlo(const double* parts, size_t n_parts, size_t rows, size_t Ev, double* out) {
    size_t w = 2 + Ev;
    std::vector<Slot> slots(w, Slot{EXP_SHIFTED, 0});
    slots[0] = {PLAIN_MAX, 0};
    std::vector<double> acc(w), tmp(w);
    for (size_t r = 0; r < rows; ++r) {
        std::copy(parts + r * w, parts + (r + 1) * w, acc.begin());
        for (size_t p = 1; p < n_parts; ++p) {
            carrier_merge(slots, acc.data(), parts + (p * rows + r) * w, tmp.data());
            acc = tmp;
        }
        for (size_t e = 0; e < Ev; ++e) out[r * Ev + e] = acc[2 + e] / acc[1];
    }
}

// rms_norm (src/nn.rs:165-169): (x * w) / sqrt(sum(x*x) * (1/n) + eps), rows x n.
void orc_rms_norm(const double* x, const double* w, size_t rows, size_t n, double eps, double* out) {
    for (size_t r = 0; r < rows; ++r) {
        double ss = 0.0;
        for (size_t i = 0; i < n; ++i) ss = ss + x[r * n + i] * x[r * n + i];
        double den = std::sqrt(ss * (1.0 / (double)n) + eps);
        for (size_t i = 0; i < n; ++i) out[r * n + i] = (x[r * n + i] * w[i]) / den;
    }
}

// eval(rms_norm(x, gamma) @ W), x [M,K], W [K,N] (or [N,K] when w_is_nk).
void orc_rmsnorm_gemm(const double* x, const double* gamma, const double* w, size_t M, size_t K, size_t N,
                      int w_is_nk, double eps, double* out) {
    std::vector<double> xn(M * K);
    orc_rms_norm(x, gamma, M, K, eps, xn.data());
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            double acc = 0.0;
            for (size_t kk = 0; kk < K; ++kk) acc = acc + xn[i * K + kk] * (w_is_nk ? w[j * K + kk] : w[kk * N + j]);
            out[i * N + j] = acc;
        }
}

// run_carrier_split of the defer-div carrier: 2 x Plain(Add) = (sum x^2, sum x*g*W),
// project = dot / sqrt(ss * (1/n) + eps)  (tests/laws.rs:620-646, src/partition.rs:2591-2608).
int orc_rmsnorm_gemm_carrier_split(const double* x, const double* gamma, const double* w, size_t M, size_t K, size_t N,
                                   int w_is_nk, double eps, size_t blocks, double* out) {
    if (blocks < 1 || blocks > K) return 1;
    std::vector<Slot> slots = {{PLAIN_ADD, 0}, {PLAIN_ADD, 0}};
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            double acc[2] = {0.0, 0.0};
            fold_split(slots, K, blocks, [&](size_t kk, double* el) {
                double xv = x[i * K + kk];
                el[0] = xv * xv;
                el[1] = (xv * gamma[kk]) * (w_is_nk ? w[j * K + kk] : w[kk * N + j]);
            }, acc);
            out[i * N + j] = acc[1] / std::sqrt(acc[0] * (1.0 / (double)K) + eps);
        }
    return 0;
}

// eval of the grouped int4 matvec (tests/metal.rs:1224-1236):
// y[b,o] = sum over the flattened (g, r) axis of (q[o,g,r] * x[b,g,r]) * s[o,g].
void orc_w4_gemv(const uint8_t* packed, const double* scales, const double* x, size_t batch, size_t n_out, size_t K,
                 size_t group, double* y) {
    size_t G = K / group;
    // Every (o, b) output adds its K terms in index order, as the interpreter's left fold does. The batch rows of
    // one weight row are independent chains, so eight of them advance together: same values, shorter wall time.
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < n_out; ++o) {
        std::vector<double> qrow(K), srow(K);
        for (size_t c = 0; c < K; ++c) {
            size_t i = o * K + c;
            qrow[c] = (double)(int)((packed[i / 2] >> ((i & 1) * 4)) & 0xF) - 8.0;
            srow[c] = scales[o * G + c / group];
        }
        for (size_t b0 = 0; b0 < batch; b0 += 8) {
            size_t nb = batch - b0 < 8 ? batch - b0 : 8;
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (nb == 8) {
                for (size_t c = 0; c < K; ++c)
                    for (size_t bb = 0; bb < 8; ++bb) acc[bb] = acc[bb] + (qrow[c] * x[(b0 + bb) * K + c]) * srow[c];
            } else {
                for (size_t c = 0; c < K; ++c)
                    for (size_t bb = 0; bb < nb; ++bb) acc[bb] = acc[bb] + (qrow[c] * x[(b0 + bb) * K + c]) * srow[c];
            }
            for (size_t bb = 0; bb < nb; ++bb) y[(b0 + bb) * n_out + o] = acc[bb];
        }
    }
}
int orc_w4_gemv_carrier_split(const uint8_t* packed, const double* scales, const double* x, size_t batch, size_t n_out,
                              size_t K, size_t group, size_t blocks, double* y) {
    if (blocks < 1 || blocks > K) return 1;
    size_t G = K / group;
    std::vector<Slot> slots = {{PLAIN_ADD, 0}};
    for (size_t o = 0; o < n_out; ++o)
        for (size_t b = 0; b < batch; ++b) {
            double acc[1] = {0.0};
            fold_split(slots, K, blocks, [&](size_t c, double* el) {
                size_t i = o * K + c;
                double qv = (double)(int)((packed[i / 2] >> ((i & 1) * 4)) & 0xF) - 8.0;
                el[0] = (qv * x[b * K + c]) * scales[o * G + c / group];
            }, acc);
            y[b * n_out + o] = acc[0];
        }
    return 0;
}

// Dense bf16-weight matvec: y[b,o] = sum_k x[b,k] * W[o,k], weights given as bf16 bits.
void orc_gemv_bf16w(const uint16_t* w, const double* x, size_t batch, size_t n_out, size_t K, double* y) {
    // per (o, b): the K terms added in index order; eight batch rows advance together (independent chains)
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < n_out; ++o) {
        std::vector<double> wrow(K);
        for (size_t c = 0; c < K; ++c) wrow[c] = bf16_widen(w[o * K + c]);
        for (size_t b0 = 0; b0 < batch; b0 += 8) {
            size_t nb = batch - b0 < 8 ? batch - b0 : 8;
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (nb == 8) {
                for (size_t c = 0; c < K; ++c)
                    for (size_t bb = 0; bb < 8; ++bb) acc[bb] = acc[bb] + x[(b0 + bb) * K + c] * wrow[c];
            } else {
                for (size_t c = 0; c < K; ++c)
                    for (size_t bb = 0; bb < nb; ++bb) acc[bb] = acc[bb] + x[(b0 + bb) * K + c] * wrow[c];
            }
            for (size_t bb = 0; bb < nb; ++bb) y[(b0 + bb) * n_out + o] = acc[bb];
        }
    }
}

// eval(argmax(x, -1)) for rows x n: first maximal index (src/ir.rs:1402-1433).
void orc_argmax(const double* x, size_t rows, size_t n, double* out) {
    for (size_t r = 0; r < rows; ++r) {
        double mx = NEG_INF;
        for (size_t i = 0; i < n; ++i) mx = cmax(mx, x[r * n + i]);
        double best = POS_INF;
        for (size_t i = 0; i < n; ++i) best = cmin(best, (x[r * n + i] < mx) ? POS_INF : (double)i);
        out[r] = best;
    }
}
// run_carrier_split of (Plain(Max), AtExtremum{key 0, Max, ties Min}); into = (x, index).
int orc_argmax_carrier_split(const double* x, size_t rows, size_t n, size_t blocks, double* out) {
    if (blocks < 1 || blocks > n) return 1;
    std::vector<Slot> slots = {{PLAIN_MAX, 0}, {AT_EXTREMUM_MAX_TIES_MIN, 0}};
    for (size_t r = 0; r < rows; ++r) {
        double acc[2] = {0.0, 0.0};
        fold_split(slots, n, blocks, [&](size_t i, double* el) { el[0] = x[r * n + i]; el[1] = (double)i; }, acc);
        out[r] = acc[1];
    }
    return 0;
}

// rope_inv_freq (src/nn.rs:197-199): exp(i * (-ln(theta) / F)).
void orc_rope_inv_freq(double theta, size_t F, double* out) {
    for (size_t i = 0; i < F; ++i) out[i] = std::exp((double)i * (-std::log(theta) / (double)F));
}
// llama3_inv_freq (examples/llama3_2.rs:95-107), constants at :28-33.
void orc_llama3_inv_freq(size_t F, double* out) {
    const double THETA = 500000.0, FACTOR = 32.0, ORIG = 8192.0, LOW = 1.0, HIGH = 4.0;
    for (size_t i = 0; i < F; ++i) {
        double inv = std::exp((double)i * (-std::log(THETA) / (double)F));
        double wave = 2.0 * 3.14159265358979323846 / inv;
        double low_wave = ORIG / LOW, high_wave = ORIG / HIGH;
        double smooth = (ORIG / wave - LOW) / (HIGH - LOW);
        double scaled = inv / FACTOR;
        double blended = (1.0 - smooth) * scaled + smooth * inv;
        out[i] = (low_wave < wave) ? scaled : ((wave < high_wave) ? inv : blended);
    }
}
// rope (src/nn.rs:176-194) over rows x D with one position per row: head_dim is
// split (pair=2, freq=D/2); out = x*cos(a) + flip_pair(x)*sign*sin(a), sign = (-1,+1).
void orc_rope(const double* x, const double* positions, const double* inv_freq, size_t rows, size_t D, double* out) {
    size_t F = D / 2;
    for (size_t r = 0; r < rows; ++r)
        for (size_t p = 0; p < 2; ++p)
            for (size_t f = 0; f < F; ++f) {
                double angle = positions[r] * inv_freq[f];
                double sign = (double)p * 2.0 - 1.0;
                double rotated = x[r * D + (1 - p) * F + f] * sign;
                out[r * D + p * F + f] = x[r * D + p * F + f] * std::cos(angle) + rotated * std::sin(angle);
            }
}

// ───────────────────────── Llama-architecture decode step ─────────────────────────
// The graph of examples/llama3_2.rs:112-253 with a leading batch axis added and a
// shared scalar position. Weights are storage-typed inputs whose meaning is their
// widened value: bf16 bits, or int4 nibbles with bf16 per-group scales (group along
// the input dimension). Caches are states declared at bf16: the value written is
// RoundTo(bf16) of the new row. `round_acts` additionally declares stored(bf16) on
// the activations a projection reads and on q, matching a bf16 boundary policy.
struct OrcLlamaCfg {
    uint64_t vocab, layers, hidden, q_heads, kv_heads, head_dim, ffn, ctx, batch;
    int32_t w4;          // 0: bf16 weights; 1: int4 + bf16 scales for the seven projections
    int32_t group;       // int4 group size along K
    int32_t round_acts;  // 1: stored(bf16) at projection inputs and q
    int32_t llama3_rope; // 1: llama3 frequency blend; 0: plain theta schedule
    int32_t w4_head;     // 1: the tied embedding / lm_head table is int4 + bf16 scales too (`embed` packed, `sembed` scales)
    int32_t norm_store;  // where stored(bf16) sits on a normed projection input (round_acts = 1):
                         //   0: on rms_norm(x) itself, bf16((x*g)/sqrt(mean(x^2)+eps));
                         //   1: on x*g, with the division deferred past the contraction (the defer-div carrier of
                         //      tests/laws.rs:620-646: slots sum x^2 and sum bf16(x*g)*W, project = dot / sqrt(ss/n + eps));
                         //   2: as 1 at every norm whose input a residual-add produces, as 0 at the one norm whose input
                         //      is the gathered embedding (layer 0's attention norm)
    double eps, theta;
};
struct OrcLlamaWeights {  // per layer arrays of pointers
    const uint16_t* embed;                 // [vocab, hidden] bf16
    const uint16_t* final_norm;            // [hidden]
    const uint16_t* const* attn_norm;      // [layers][hidden]
    const uint16_t* const* mlp_norm;
    const void* const* wq; const void* const* wk; const void* const* wv; const void* const* wo;
    const void* const* wgate; const void* const* wup; const void* const* wdown;
    const uint16_t* const* sq; const uint16_t* const* sk; const uint16_t* const* sv; const uint16_t* const* so;
    const uint16_t* const* sgate; const uint16_t* const* sup; const uint16_t* const* sdown;
    const uint16_t* sembed;                // [vocab, hidden/group] bf16 scales of an int4 table (w4_head)
};
struct OrcLlama {
    OrcLlamaCfg cfg;
    OrcLlamaWeights w;
    std::vector<double> kcache, vcache;  // [layers][batch][kv][ctx][hd] and [layers][batch][kv][hd][ctx]
    std::vector<double> inv_freq;
    std::vector<double> logits;
};

static void project(const OrcLlama* m, const void* w, const uint16_t* s, const std::vector<double>& x, size_t batch,
                    size_t n_out, size_t K, std::vector<double>& y, int force_w4 = -1) {
    y.assign(batch * n_out, 0.0);
    if (force_w4 >= 0 ? force_w4 != 0 : m->cfg.w4 != 0) {
        std::vector<double> sc((n_out * K) / m->cfg.group);
        orc_from_bf16_bits(s, sc.data(), sc.size());
        orc_w4_gemv((const uint8_t*)w, sc.data(), x.data(), batch, n_out, K, m->cfg.group, y.data());
    } else {
        orc_gemv_bf16w((const uint16_t*)w, x.data(), batch, n_out, K, y.data());
    }
}
static void maybe_round(const OrcLlama* m, std::vector<double>& v) {
    if (m->cfg.round_acts) for (double& x : v) x = round_bf16(x);
}
// The normed input of a projection and the factor its outputs are still to be divided by.
// norm_store 0: xn = stored(rms_norm(x, g)), den = 1. norm_store 1: xn = stored(x * g), den[b] = sqrt(mean(x^2) + eps):
// the contraction runs on x*g and each output row is divided once afterwards (defer-div).
static void normed_input(const OrcLlama* m, const std::vector<double>& x, const std::vector<double>& gamma, size_t B, size_t Hd,
                         std::vector<double>& xn, std::vector<double>& den, bool after_gather = false) {
    xn.resize(B * Hd);
    den.assign(B, 1.0);
    if (m->cfg.norm_store == 0 || (m->cfg.norm_store == 2 && after_gather)) {
        orc_rms_norm(x.data(), gamma.data(), B, Hd, m->cfg.eps, xn.data());
    } else {
        for (size_t b = 0; b < B; ++b) {
            double ss = 0.0;
            for (size_t i = 0; i < Hd; ++i) ss = ss + x[b * Hd + i] * x[b * Hd + i];
            den[b] = std::sqrt(ss * (1.0 / (double)Hd) + m->cfg.eps);
            for (size_t i = 0; i < Hd; ++i) xn[b * Hd + i] = x[b * Hd + i] * gamma[i];
        }
    }
    maybe_round(m, xn);
}
static void divide_rows(std::vector<double>& y, const std::vector<double>& den, size_t B, size_t n) {
    for (size_t b = 0; b < B; ++b)
        if (den[b] != 1.0) for (size_t i = 0; i < n; ++i) y[b * n + i] = y[b * n + i] / den[b];
}

OrcLlama* orc_llama_create(const OrcLlamaCfg* cfg, const OrcLlamaWeights* w) {
    OrcLlama* m = new OrcLlama();
    m->cfg = *cfg; m->w = *w;
    size_t per = cfg->layers * cfg->batch * cfg->kv_heads * cfg->ctx * cfg->head_dim;
    m->kcache.assign(per, 0.0); m->vcache.assign(per, 0.0);
    m->inv_freq.resize(cfg->head_dim / 2);
    if (cfg->llama3_rope) orc_llama3_inv_freq(cfg->head_dim / 2, m->inv_freq.data());
    else orc_rope_inv_freq(cfg->theta, cfg->head_dim / 2, m->inv_freq.data());
    return m;
}
void orc_llama_destroy(OrcLlama* m) { delete m; }
double* orc_llama_kcache(OrcLlama* m) { return m->kcache.data(); }
double* orc_llama_vcache(OrcLlama* m) { return m->vcache.data(); }
const double* orc_llama_logits(OrcLlama* m) { return m->logits.data(); }

// One decode step for every batch row at the shared `position`. tokens_in/out: [batch].
int orc_llama_step(OrcLlama* m, const int32_t* tokens_in, int64_t position, int32_t* tokens_out) {
    const OrcLlamaCfg& c = m->cfg;
    size_t B = c.batch, Hd = c.hidden, D = c.head_dim, Hq = c.q_heads, Hk = c.kv_heads, F = c.ffn, T = c.ctx;
    size_t rep = Hq / Hk;
    if ((size_t)position >= T) return 1;
    std::vector<double> x(B * Hd), gamma(Hd), xn, den, q, k, v, tmp, att(B * Hd), proj, gate, up, h;
    for (size_t b = 0; b < B; ++b) {  // Gather rounds its index (src/interp.rs:378-379)
        size_t tok = (size_t)std::llround((double)tokens_in[b]);
        if (tok >= c.vocab) return 2;
        if (c.w4_head) {   // an I4 input means its widened values: (nibble - 8) * scale of its group
            const uint8_t* packed = (const uint8_t*)m->w.embed;
            for (size_t i = 0; i < Hd; ++i) {
                size_t e = tok * Hd + i;
                double qv = (double)(int)((packed[e / 2] >> ((e & 1) * 4)) & 0xF) - 8.0;
                x[b * Hd + i] = qv * bf16_widen(m->w.sembed[tok * (Hd / c.group) + i / c.group]);
            }
        } else {
            orc_from_bf16_bits(m->w.embed + tok * Hd, &x[b * Hd], Hd);
        }
    }
    std::vector<double> pos(1, (double)position);
    for (size_t l = 0; l < c.layers; ++l) {
        orc_from_bf16_bits(m->w.attn_norm[l], gamma.data(), Hd);
        normed_input(m, x, gamma, B, Hd, xn, den, l == 0);
        project(m, m->w.wq[l], c.w4 ? m->w.sq[l] : nullptr, xn, B, Hq * D, Hd, q);
        project(m, m->w.wk[l], c.w4 ? m->w.sk[l] : nullptr, xn, B, Hk * D, Hd, k);
        project(m, m->w.wv[l], c.w4 ? m->w.sv[l] : nullptr, xn, B, Hk * D, Hd, v);
        divide_rows(q, den, B, Hq * D); divide_rows(k, den, B, Hk * D); divide_rows(v, den, B, Hk * D);
        // rope on q and k: rows are (batch, head), all at the shared position
        std::vector<double> posq(B * Hq, (double)position), posk(B * Hk, (double)position);
        tmp.resize(q.size()); orc_rope(q.data(), posq.data(), m->inv_freq.data(), B * Hq, D, tmp.data()); q = tmp;
        tmp.resize(k.size()); orc_rope(k.data(), posk.data(), m->inv_freq.data(), B * Hk, D, tmp.data()); k = tmp;
        maybe_round(m, q);
        // update_cache (src/nn.rs:208-212) at bf16 storage; V cache is [kv, hd, seq]
        double* kc = &m->kcache[l * B * Hk * T * D];
        double* vc = &m->vcache[l * B * Hk * T * D];
        for (size_t b = 0; b < B; ++b)
            for (size_t hk = 0; hk < Hk; ++hk)
                for (size_t d = 0; d < D; ++d) {
                    kc[((b * Hk + hk) * T + position) * D + d] = round_bf16(k[(b * Hk + hk) * D + d]);
                    vc[((b * Hk + hk) * D + d) * T + position] = round_bf16(v[(b * Hk + hk) * D + d]);
                }
        // attention over the whole cache with the -inf visibility mask
        // (examples/llama3_2.rs:175-180): scores for hidden positions are -inf, exp -> 0.
        double scale = 1.0 / std::sqrt((double)D);
#pragma omp parallel for collapse(2) schedule(static)
        for (size_t b = 0; b < B; ++b)
            for (size_t hq = 0; hq < Hq; ++hq) {
                size_t hk = hq / rep;
                const double* Q = &q[(b * Hq + hq) * D];
                std::vector<double> sc(T), ex(T);
                for (size_t t = 0; t < T; ++t) {
                    const double* K = &kc[((b * Hk + hk) * T + t) * D];
                    double acc = 0.0;
                    for (size_t d = 0; d < D; ++d) acc = acc + Q[d] * K[d];
                    acc = acc * scale;
                    sc[t] = acc + (((double)t < (double)position + 1.0) ? 0.0 : NEG_INF);
                }
                double mx = NEG_INF;
                for (size_t t = 0; t < T; ++t) mx = cmax(mx, sc[t]);
                double z = 0.0;
                for (size_t t = 0; t < T; ++t) { ex[t] = std::exp(sc[t] - mx); z = z + ex[t]; }
                for (size_t d = 0; d < D; ++d) {
                    const double* V = &vc[((b * Hk + hk) * D + d) * T];
                    double acc = 0.0;
                    for (size_t t = 0; t < T; ++t) acc = acc + (ex[t] / z) * V[t];
                    att[b * Hd + hq * D + d] = acc;
                }
            }
        std::vector<double> attr = att; maybe_round(m, attr);
        project(m, m->w.wo[l], c.w4 ? m->w.so[l] : nullptr, attr, B, Hd, Hd, proj);
        for (size_t i = 0; i < B * Hd; ++i) x[i] = x[i] + proj[i];
        orc_from_bf16_bits(m->w.mlp_norm[l], gamma.data(), Hd);
        normed_input(m, x, gamma, B, Hd, xn, den);
        project(m, m->w.wgate[l], c.w4 ? m->w.sgate[l] : nullptr, xn, B, F, Hd, gate);
        project(m, m->w.wup[l], c.w4 ? m->w.sup[l] : nullptr, xn, B, F, Hd, up);
        divide_rows(gate, den, B, F); divide_rows(up, den, B, F);
        h.resize(B * F);
        for (size_t i = 0; i < B * F; ++i) {  // silu(g) * up  (src/ir.rs:1500-1509)
            double sig = 1.0 / (1.0 + std::exp(-gate[i]));
            h[i] = (gate[i] * sig) * up[i];
        }
        maybe_round(m, h);
        project(m, m->w.wdown[l], c.w4 ? m->w.sdown[l] : nullptr, h, B, Hd, F, proj);
        for (size_t i = 0; i < B * Hd; ++i) x[i] = x[i] + proj[i];
    }
    orc_from_bf16_bits(m->w.final_norm, gamma.data(), Hd);
    normed_input(m, x, gamma, B, Hd, xn, den);
    project(m, m->w.embed, c.w4_head ? m->w.sembed : nullptr, xn, B, c.vocab, Hd, m->logits, c.w4_head ? 1 : 0);
    divide_rows(m->logits, den, B, c.vocab);
    std::vector<double> idx(B);
    orc_argmax(m->logits.data(), B, c.vocab, idx.data());
    for (size_t b = 0; b < B; ++b) tokens_out[b] = (int32_t)idx[b];
    return 0;
}

}  // extern "C"
