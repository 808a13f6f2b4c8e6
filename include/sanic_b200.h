/*
 * sanic_b200 — C ABI of the B200 (sm_100a) backend for sanic's derived carriers.
 *
 * This is the drop-in boundary: what a `Backend` implementation on the reference
 * side (src/compile.rs:87-108) binds instead of src/emit_metal.rs + src/metal.rs.
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an
 * int32 status (0 = OK), never throws and never aborts. `sanic_last_error(ctx)`
 * gives the text of the last failure on that context.
 *
 * All device pointers are CUdeviceptr-compatible addresses in the context's
 * device. All work is enqueued on the caller's stream (a cudaStream_t passed as
 * void*; NULL = the default stream). One context per device per process; calls
 * on one context are not thread-safe.
 *
 * Paths cited below are relative to the reference project.
 */
#ifndef SANIC_B200_H
#define SANIC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sanic_ctx sanic_ctx;

/* Status codes. RunError / CompileError of src/compile.rs:18-78 map onto these. */
enum {
    SANIC_OK = 0,
    SANIC_ERR_INVALID = 1,      /* CompileError::InvalidInput / RunError::Shape: bad argument */
    SANIC_ERR_CUDA = 2,         /* RunError::Backend: a CUDA call failed */
    SANIC_ERR_UNSUPPORTED = 3,  /* CompileError::Backend: no kernel for this carrier structure */
    SANIC_ERR_TIMEOUT = 4,      /* a bounded device-side wait ran out */
    SANIC_ERR_NCCL = 5,
    SANIC_ERR_DTYPE = 6,        /* RunError::Dtype */
    SANIC_ERR_NOMEM = 7,
    SANIC_ERR_MISSING_INPUT = 8,    /* RunError::MissingInput */
    SANIC_ERR_UNKNOWN_INPUT = 9,    /* RunError::UnknownInput */
    SANIC_ERR_DUPLICATE_INPUT = 10, /* RunError::DuplicateInput */
    SANIC_ERR_SHAPE = 11,           /* RunError::Shape */
    SANIC_ERR_FEEDBACK = 12         /* RunError::Feedback */
};

/* Storage widths (src/scalar.rs:181-201). */
enum { SANIC_F32 = 1, SANIC_F16 = 2, SANIC_BF16 = 3, SANIC_U32 = 4, SANIC_I4 = 5,
       SANIC_F64 = 6 /* an arithmetic width only (accum_dtype); no buffer is stored at it */ };

/* ── context and memory: replaces MetalDevice open/alloc/read (src/metal.rs:149-490) ── */
int32_t sanic_cuda_open(int32_t ordinal, sanic_ctx** out);
int32_t sanic_cuda_close(sanic_ctx* ctx);
const char* sanic_last_error(sanic_ctx* ctx);
const char* sanic_version(void);

/* Hardware facts only, as Backend::specs (src/compile.rs:91-93, src/cost.rs:33-60). */
typedef struct {
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int32_t max_smem_per_block;
    int32_t l2_bytes;
    int32_t warp;            /* SIMD width (src/plan.rs:458) */
    uint64_t hbm_bytes;
    double hbm_gbs_nominal;
    double bf16_tflops_nominal;
} sanic_device_specs;
int32_t sanic_specs(sanic_ctx* ctx, sanic_device_specs* out);

/* Measured facts next to the datasheet ones: what a fitted DeviceSpecs carries (src/cost.rs:62-119) and what the
 * reference's in-context timing measures (src/compile.rs:1348-1630). Both probes are tiny, bounded kernels.
 * sanic_probe_sfu: `ex2.approx` per clock per SM with `warps_per_sm` resident warps (one CTA per SM); mode 0 = the
 * exponentials alone, 1 = + the scale-and-shift FMA per element, 2 = + the row-sum add, 3 = + the bf16x2 pack: the inner
 * loop of the online-softmax warps; 4 / 5 = mode 3 with every fourth / second pair of exponentials on the FMA pipe (cubic);
 * 6-8 = a pair's exponentials as one packed f16x2 instruction (6: with the scale FMA and the conversion only, 7: + unpack,
 * row sum and bf16x2 pack, 8: + unpack and row sum, result kept as f16); 9 / 10 = mode 3 with the row maximum in the same loop
 * (one three-input max per pair / two two-input ones). *clk_per_128_per_warp (optional) is the raw figure: clocks per 128 elements per lane.
 * sanic_probe_stream: GB/s of a read-only sweep of `buffer` (best of `repeats`), the rate an HBM-bound fold is held to. */
int32_t sanic_probe_sfu(sanic_ctx* ctx, int32_t warps_per_sm, int32_t mode, int32_t iters, void* stream, double* exp_per_clk_per_sm,
                        double* clk_per_128_per_warp);
int32_t sanic_probe_stream(sanic_ctx* ctx, const void* buffer, size_t bytes, int32_t repeats, void* stream, double* gb_per_s);

int32_t sanic_alloc(sanic_ctx* ctx, size_t bytes, void** dptr);
int32_t sanic_free(sanic_ctx* ctx, void* dptr);
int32_t sanic_upload(sanic_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes, void* stream);
int32_t sanic_download(sanic_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes, void* stream);
int32_t sanic_memset(sanic_ctx* ctx, void* dptr, int32_t byte, size_t bytes, void* stream);
int32_t sanic_sync(sanic_ctx* ctx, void* stream);
/* Host-side failure injection (the reference surfaces device failures as Err(String) from run_graph_timed,
 * src/metal.rs:686-705; there is no device-side injector here): writes `code` into the context's status word exactly as a
 * kernel whose bounded wait ran out would, so the next sanic_sync returns the matching error and clears the word.
 * Codes: 1-29 mbarrier waits of the tensor-core kernels, 31-33 persistent step (grid barrier, ring full, ring empty),
 * 41+q peer flag of rank q, 51 gather index, 52 decode length clamp. No kernel is launched and nothing on the device is disturbed. */
int32_t sanic_status_inject(sanic_ctx* ctx, int32_t code);

/* ── carrier structure: what the emitter keys kernel choice on (src/derive.rs:519-530) ── */
enum { SANIC_SLOT_PLAIN_ADD = 1, SANIC_SLOT_PLAIN_MAX = 2, SANIC_SLOT_PLAIN_MIN = 3,
       SANIC_SLOT_EXP_SHIFTED = 4, SANIC_SLOT_AT_EXTREMUM = 5 };
typedef struct {
    int32_t n_slots;
    int32_t kind[4];      /* SANIC_SLOT_* */
    int32_t ref[4];       /* max_slot (EXP_SHIFTED) or key_slot (AT_EXTREMUM) */
    int32_t leaf_dtype;   /* storage of the streamed leaf: SANIC_F32 / SANIC_BF16 / SANIC_I4 */
    int32_t in_body_contraction; /* 1 when a leaf is itself a contraction (QK^T in the fold body) */
    int32_t deferred_div; /* 1 when project divides by a function of another slot (defer-div) */
} sanic_carrier_desc;
/* Kernel families the emitter can select (the K1..K4 rows of src/emit_metal.rs). */
enum { SANIC_KERNEL_NONE = 0, SANIC_KERNEL_ONLINE_SOFTMAX_FOLD = 1, SANIC_KERNEL_DEFERRED_NORM_CONTRACTION = 2,
       SANIC_KERNEL_PLAIN_CONTRACTION = 3, SANIC_KERNEL_GROUPED_I4_CONTRACTION = 4, SANIC_KERNEL_EXTREMUM_INDEX = 5 };
/* Maps a carrier to a kernel family by slot kinds and leaves only, never by an
 * operation name (the layering rule of tests/structure.rs:153-203; the analogue of
 * the structural matching in src/emit_metal.rs:457-505). SANIC_ERR_UNSUPPORTED if none. */
int32_t sanic_emit_select(const sanic_carrier_desc* carrier, int32_t* kernel_family);

/* ── K2a: online-softmax fold (m, l, o) — replaces the cooperative fold kernel the
 *    Metal emitter generates for this carrier (src/emit_metal.rs:760-1101) ── */
typedef struct {
    const void* q; const void* k; const void* v; void* out;
    int32_t batch, q_heads, kv_heads;      /* q head h reads kv head h / (q_heads/kv_heads) (src/nn.rs:107-151) */
    int32_t q_len, kv_len, head_dim, v_dim;
    int32_t causal;                        /* where(i < j, -1e30, 0) (src/ir.rs:1511-1526) */
    int32_t window;                        /* 0 = none; else query s sees keys s-window+1..s (tests/movement.rs:294-345) */
    float scale;
    const float* mask;                     /* optional additive mask [q_len, kv_len] (f32 path only) */
    int32_t out_dtype;                     /* SANIC_F32 or SANIC_BF16 */
    int32_t accum_dtype;                   /* f32 path only. 0 / SANIC_F32: f32 arithmetic. SANIC_F64: scores, exponentials and
                                              the (m, l, o) carrier in f64, rounded once at the store: the plain relative error
                                              against the f64 interpreter (src/interp.rs:270-518) stays at f32 rounding level even
                                              where an output is a near cancellation of its terms */
} sanic_attn_params;
/* f32 storage, f32 CUDA-core arithmetic: q [B,Hq,L,E], k [B,Hkv,S,E], v [B,Hkv,S,Ev], out [B,Hq,L,Ev]. */
int32_t sanic_attn_fwd_f32(sanic_ctx* ctx, const sanic_attn_params* p, void* stream);
/* bf16 storage, tcgen05 contractions with accumulators in tensor memory, f32 carrier in registers. E = Ev = 64 (the
 * head size of the prefill configuration); any other head size is refused with SANIC_ERR_UNSUPPORTED. */
int32_t sanic_attn_fwd_bf16(sanic_ctx* ctx, const sanic_attn_params* p, void* stream);
/* One launch of the same kernel with clock counters on in CTA 0 (a finer view than the per-kernel times of the reference's
 * SANIC_DEBUG=4, src/compile.rs:1147-1346). For query tile t (0, 1) of the CTA's work items, from the softmax warp of the
 * tile's rows 0-31, out[10t + i] = clocks spent, summed over its key tiles: [0] waiting for the scores, [1] loading them
 * and taking the row maximum, [2] the first 64 exponentials, [3] waiting for the previous PV product, [4] rescaling O,
 * [5] storing P and the second 64 exponentials, [6] the store wait and the arrival, [7] epilogues and item switches;
 * [8] key tiles folded, [9] clocks over all. For the tile's MMA thread, m = 20 + 8t: out[m] its polls, [m+1] of those
 * without anything to issue, [m+2] its clocks, [m+3] score tiles issued, and its clocks in [m+4] barrier tests and idle
 * sleeps, [m+5] issuing the score products (four MMAs and a commit each), [m+6] the value products (eight MMAs and two
 * commits), [m+7] item switches. out (36 words, host memory) is written; the attention output too. Synchronises. */
int32_t sanic_attn_fwd_bf16_profile(sanic_ctx* ctx, const sanic_attn_params* p, void* stream, uint64_t* out);

/* Split-KV decode (one query token per sequence). Stage 1 folds contiguous chunks of
 * the key axis into raw (m, l, o) accumulators exactly as run_carrier_split chunks it
 * (src/interp.rs:597-631); stage 2 merges them with the derived combine
 * (src/derive.rs:1700-1713) and either projects o/l or exports the merged carrier. */
typedef struct {
    const void* q;            /* [B, Hq, D] bf16 */
    const void* k;            /* bf16; element strides below; head_dim contiguous */
    const void* v;            /* bf16; v_transposed=0: [.., seq, D] ; 1: [.., D, seq] (examples/llama3_2.rs:160-173) */
    int64_t k_batch_stride, k_head_stride, k_seq_stride;
    int64_t v_batch_stride, v_head_stride, v_row_stride;  /* row = seq (v_transposed=0) or dim (1) */
    int32_t v_transposed;
    int32_t batch, q_heads, kv_heads, head_dim;
    int32_t kv_len;           /* visible prefix length when kv_len_dev is NULL */
    const int32_t* kv_len_dev;/* optional: device scalar holding position; visible length = *kv_len_dev + 1 */
    int32_t window;           /* 0 = none */
    int32_t n_splits;         /* chunks of the key axis per (batch, kv head) */
    float scale;
    float* partials;          /* scratch of sanic_attn_decode_scratch_bytes() bytes, zero-filled once before its
                                 first use: raw accumulators [B*Hq, n_splits, 2 + D] then one ticket per (batch, kv head) */
    float* carrier_out;       /* optional [B*Hq, 2 + D] f32: merged raw accumulator (m natural-log units, l, o) */
    void* out;                /* optional projected output [B, Hq, D] */
    int32_t out_dtype;        /* SANIC_F32 or SANIC_BF16 */
    int32_t kv_cap;           /* extent of the key axis of k and v (the cache's sequence extent). Required (>= 1) with
                                 kv_len_dev, checked against the strides on the host; the kernel never reads a key at or
                                 beyond it: a device-side length outside [1, kv_cap] is clamped and the next sanic_sync
                                 fails with SANIC_ERR_INVALID (code 52). 0 with a host kv_len = unchecked */
} sanic_decode_params;
int32_t sanic_attn_decode_splitkv(sanic_ctx* ctx, const sanic_decode_params* p, void* stream);
size_t sanic_attn_decode_scratch_bytes(int32_t batch, int32_t q_heads, int32_t head_dim, int32_t n_splits);
/* Suggested number of chunks for this device and shape (a multiple of the SM count in CTAs). */
int32_t sanic_attn_decode_suggest_splits(sanic_ctx* ctx, int32_t batch, int32_t kv_heads, int32_t head_dim, int64_t kv_len);

/* The same fold with the (batch, kv head, key tile) space cut into one contiguous range per CTA of an exactly resident
 * grid (stream-K), so that no partial last wave is paid when the key axis is short for the device (a per-device slice of a
 * sharded cache). p->n_splits is the number of partial slots per row of `partials`: at least
 * sanic_attn_decode_streamk_slots(); the scratch layout and size are those of sanic_attn_decode_splitkv for that n_splits.
 * The chunk boundaries differ from the fixed-chunk form's; any chunking merges to the same value (src/interp.rs:538-554). */
int32_t sanic_attn_decode_streamk(sanic_ctx* ctx, const sanic_decode_params* p, void* stream);
int32_t sanic_attn_decode_streamk_slots(sanic_ctx* ctx, int32_t batch, int32_t kv_heads, int32_t head_dim);

/* Same fold for callers that cannot allocate device memory. This entry point has no counterpart in
 * the reference. Some hosts of this library may not call cudaMalloc at the point where they decode:
 * a latency-critical serving loop where an allocation would synchronise the device, plugins that are handed a fixed arena by their framework, and
 * processes whose memory is fully budgeted up front. For them the split-KV scratch lives in a static
 * device array inside the library (4 MiB of partial accumulators plus 4096 ticket counters, held on
 * every device that loads the library until the process exits). `p->partials` is ignored; inputs and
 * outputs are still the caller's. The call fails with SANIC_ERR_INVALID, and says so, when
 * batch*q_heads*n_splits*(head_dim+2) floats exceed sanic_attn_decode_static_scratch_capacity() bytes
 * or batch*kv_heads exceeds 4096. It calls no cudaMalloc, cudaFree or allocating library routine.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 * first call before starting any stream capture. All calls share the one array and it keeps the last
 * call's contents: the counters are cleared on the stream at every call, and two calls that overlap
 * on the GPU (different streams, or different threads) race on it. */
int32_t sanic_attn_decode_splitkv_static(sanic_ctx* ctx, const sanic_decode_params* p, void* stream);
size_t sanic_attn_decode_static_scratch_capacity(void);

/* Stage 2 alone: merge n_parts raw accumulators [n_parts, rows, 2+D] left to right and
 * project. This is the cross-device merge of interp::run_carrier_split (src/interp.rs:632-639). */
int32_t sanic_carrier_merge(sanic_ctx* ctx, const float* parts, int32_t n_parts, int32_t rows, int32_t head_dim,
                            float* carrier_out, void* out, int32_t out_dtype, void* stream);

/* ── K2b: deferred-normaliser contraction (RMSNorm-fused GEMM), tcgen05 + TMA.
 *    y = (sum_k x*g*W) / sqrt(sum_k x^2 / K + eps)  (tests/laws.rs:620-646, src/partition.rs:2591-2608) ── */
typedef struct {
    const void* x;      /* [M, K] bf16 */
    const void* gamma;  /* [K] bf16 */
    const void* w;      /* w_is_nk=1: [N, K] (checkpoint-native [out,in], examples/llama3_2.rs:85-90); 0: [K, N] */
    void* y;            /* [M, N] */
    int32_t M, N, K;
    int32_t w_is_nk;
    float eps;
    int32_t out_dtype;  /* SANIC_BF16 or SANIC_F32 */
} sanic_gemm_rmsnorm_params;
int32_t sanic_gemm_rmsnorm(sanic_ctx* ctx, const sanic_gemm_rmsnorm_params* p, void* stream);
/* For weights that are bound once (a stateful program, src/graph.rs:231-356): w_out = bf16(W * g) along K, the
 * rewrite sum (x*g)*W = sum x*(g*W). sanic_gemm_rmsnorm with gamma == NULL then takes w_out as W: the activations go
 * to the tensor core as loaded and only sum x^2 is taken from them, which removes the per-stage transform from the
 * pipeline's latency. One factor is rounded to bf16 either way (x*g there, g*W here). */
/* One launch of the 256 x 256 pair tile with A brought in through registers, with clock counters on in the roles of SM pair 0
 * (a finer view than the per-kernel times of the reference's SANIC_DEBUG=4, src/compile.rs:1147-1346): out[0] k-blocks the
 * MMA thread issued, [1] its clocks over its loop, [2] of those, clocks reading the progress counters, [3] counter reads,
 * [4] clocks waiting for a free accumulator; [5] the B producer's clocks waiting for a free slot; transform warp 0 of the
 * leader [6..11] and of the peer [12..17]: its k-blocks, then clocks in arithmetic (including the wait for its loads),
 * waiting for the slot, storing, in the proxy fence, in the arrival. y is written as by sanic_gemm_rmsnorm. Synchronises. */
int32_t sanic_gemm_rmsnorm_pair_profile(sanic_ctx* ctx, const sanic_gemm_rmsnorm_params* p, void* stream, uint64_t* out);
int32_t sanic_gemm_prescale_weights(sanic_ctx* ctx, const void* gamma, const void* w, void* w_out, int32_t N, int32_t K,
                                    int32_t w_is_nk, void* stream);

/* ── K2c / plain contraction at decode batch sizes: y[b,o] = sum_k x[b,k] * W[o,k].
 *    Weights bf16, or int4 nibbles (q+8, low nibble = even element, src/emit_metal.rs:179-181)
 *    with a bf16 scale per `group` inputs (tests/metal.rs:1224-1236). Up to three weight
 *    segments share one launch (q/k/v projections); a segment pair can be combined as
 *    silu(a)*b (src/ir.rs:1500-1509); the result can be added to a residual. ── */
enum { SANIC_EPI_STORE = 0, SANIC_EPI_RESIDUAL_ADD = 1, SANIC_EPI_SILU_MUL = 2, SANIC_EPI_ROPE_CACHE = 3 };
typedef struct {
    const void* x;            /* [batch, K] bf16 activations */
    int32_t batch, K;
    int32_t weight_dtype;     /* SANIC_BF16 or SANIC_I4 */
    int32_t group;            /* int4 group size along K (64) */
    int32_t n_segments;       /* 1..3 */
    const void* w[3];         /* [rows_i, K] bf16 or [rows_i, K/2] bytes */
    const void* scales[3];    /* [rows_i, K/group] bf16 (int4 only) */
    int32_t rows[3];
    void* out[3];             /* [batch, rows_i] */
    int32_t out_dtype;        /* SANIC_F32 or SANIC_BF16 */
    int32_t epilogue;         /* SANIC_EPI_* ; SILU_MUL needs n_segments == 2 with equal rows, result in out[0] */
    const float* residual;    /* [batch, rows_0] f32 for RESIDUAL_ADD (may alias out[0] when out is f32) */
    /* Optional inlined producer cone (the partitioner's leaf inlining, src/partition.rs:860-1016): when norm_x is
     * set, the activations are bf16((norm_x * norm_gamma) / sqrt(mean(norm_x^2) + norm_eps)) computed inside the
     * kernel from the f32 rows norm_x [batch, K], and `x` is ignored. */
    const float* norm_x; const void* norm_gamma; float norm_eps;
    /* ROPE_CACHE epilogue (three segments q, k, v of one decode step): rotate-half RoPE at *rope_position on q and
     * k, q -> rope_q_out bf16 [B,Hq,D], k -> row *rope_position of the K cache [B,Hkv,ctx,D], v -> column
     * *rope_position of the V cache [B,Hkv,D,ctx] (src/nn.rs:176-212); out[] is ignored. */
    const float* rope_table; const int32_t* rope_position; void* rope_q_out; void* rope_k_cache; void* rope_v_cache;
    int32_t rope_q_heads, rope_kv_heads, rope_head_dim, rope_ctx;
    /* Deferred normaliser across two contractions (the defer-div carrier, tests/laws.rs:620-646, with its two sums produced
     * where they are cheapest). Producer, RESIDUAL_ADD epilogue with f32 output only: besides y = residual + W x the epilogue
     * writes nx_out[b, row] = bf16(y * nx_gamma[row]) (the next contraction's activations, stored(bf16) on x*g) and, per
     * 16-row tile t, nx_partial[b, t] = sum of y^2 over the tile's rows ([batch, rows_0 / 16] f32). Consumer, any epilogue,
     * no inlined norm: every output is multiplied by 1 / sqrt(sum_t ds_partial[b, t] / K + ds_eps) before the epilogue acts on
     * it (ds_tiles = K / 16; the sum runs in a fixed order). All NULL / 0: off. */
    void* nx_out; const void* nx_gamma; float* nx_partial;
    const float* ds_partial; int32_t ds_tiles; float ds_eps;
} sanic_gemv_params;
int32_t sanic_gemv(sanic_ctx* ctx, const sanic_gemv_params* p, void* stream);

/* ── K2d: extremal-key payload fold (first-max index), u32 saturating store
 *    (src/derive.rs:1714-1735, src/emit_metal.rs:186-190) ── */
int32_t sanic_argmax(sanic_ctx* ctx, const float* x, int32_t rows, int32_t n, uint32_t* out_index,
                     float* scratch /* >= rows*2*256 floats */, void* stream);

/* ── K3: pointwise stages (src/emit_metal.rs:1118-1178) ── */
/* xn = bf16((x * g) / sqrt(mean(x^2) + eps)) for rows of f32 x (src/nn.rs:165-169). */
int32_t sanic_rmsnorm(sanic_ctx* ctx, const float* x, const void* gamma_bf16, int32_t rows, int32_t n, float eps,
                      void* out_bf16, void* stream);
/* Embedding gather: out[b,:] = widen(table[token[b],:]) (Stage::Gather, src/partition.rs:2938-2946). */
int32_t sanic_embed_gather(sanic_ctx* ctx, const void* table_bf16, const int32_t* tokens, int32_t batch, int32_t hidden,
                           int32_t vocab, float* out, void* stream);
/* The same gather from an int4 group-quantised table (config 4's int4 variant quantises the tied embedding too):
 * table [vocab, hidden/2] nibbles (q + 8, low nibble = even element, src/emit_metal.rs:179-181), scales [vocab,
 * hidden/group] bf16; out[b, i] = (nibble - 8) * scale[token[b], i / group] (the widened value an I4 input means). */
int32_t sanic_embed_gather_w4(sanic_ctx* ctx, const void* table_i4, const void* scales_bf16, const int32_t* tokens, int32_t batch,
                              int32_t hidden, int32_t vocab, int32_t group, float* out, void* stream);
/* cos/sin table for RoPE: table[pos][f] = (cos(pos*inv_freq[f]), sin(pos*inv_freq[f])), angles and
 * sincos evaluated in f64 on the device, stored f32. inv_freq is a HOST array of n_freq doubles: the
 * schedule (plain theta^(-i/F) of src/nn.rs:197-199, or the llama3 blend of examples/llama3_2.rs:95-107)
 * is the caller's policy, as in the reference. */
int32_t sanic_rope_table(sanic_ctx* ctx, const double* inv_freq_host, int32_t n_freq, int32_t n_pos, float* table,
                         void* stream);
/* Rotate-half RoPE (src/nn.rs:176-194) on bf16 rows [rows, seq, D] with position = pos0 + s; in place allowed. */
int32_t sanic_rope_bf16(sanic_ctx* ctx, const void* x, void* out, int64_t rows, int32_t seq, int32_t head_dim,
                        const float* table, int32_t pos0, void* stream);
/* Decode-step RoPE + in-place cache row write (src/nn.rs:208-212, src/graph.rs:127-160):
 * qkv f32 [B, (Hq+2*Hkv)*D] -> q_out bf16 [B,Hq,D] (roped), K cache [B,Hkv,ctx,D] row pos <- bf16(rope(k)),
 * V cache [B,Hkv,D,ctx] column pos <- bf16(v). Position read from the device scalar. */
typedef struct {
    const float* q; const float* k; const float* v;   /* [B, Hq*D], [B, Hkv*D], [B, Hkv*D] f32 */
    void* q_out; void* k_cache; void* v_cache;
    const float* table;         /* [ctx][D/2][2] from sanic_rope_table */
    const int32_t* position;    /* device scalar */
    int32_t batch, q_heads, kv_heads, head_dim, ctx;
} sanic_rope_cache_params;
int32_t sanic_rope_cache_write(sanic_ctx* ctx, const sanic_rope_cache_params* p, void* stream);
/* position += 1 on the device, so a captured step replays without host writes. */
int32_t sanic_advance_position(sanic_ctx* ctx, int32_t* position, void* stream);

/* Non-finite values (NaN, +-inf) of a float buffer, counted: the check behind SANIC_NANSCAN=1, under which every run and
 * replayed step of a schedule scans the float buffers the runtime owns and names the first offender in its error
 * (the reference's pass: src/compile.rs:1261-1275). Synchronises `stream`. SANIC_DEBUG=1/2/3 (read once, as
 * src/lib.rs:38-46): one line per captured replay / per replayed step with its device time / the stage list. */
int32_t sanic_count_nonfinite(sanic_ctx* ctx, const void* dptr, size_t n, int32_t dtype, void* stream, uint32_t* count);

/* ── K4: typed load/store helpers exposed for bit-exactness tests (src/emit_metal.rs:123-232) ── */
int32_t sanic_round_to_bf16(sanic_ctx* ctx, const float* x, size_t n, uint16_t* out_bits, void* stream);
int32_t sanic_store_u32_saturating(sanic_ctx* ctx, const float* x, size_t n, uint32_t* out, void* stream);
int32_t sanic_w4_unpack(sanic_ctx* ctx, const uint8_t* packed, size_t n_elems, float* out, void* stream);

/* ── K1 / K2 / K3 generic: any carrier, given as expression programs, rendered to CUDA C and compiled at run
 *    time for sm_100a. The fallback for carriers no specialised kernel matches and the pointwise kernel of
 *    elementwise cones: the role of emit_fused_metal_with (scalar fold, src/emit_metal.rs:626-736), the
 *    cooperative fold (:760-1101) and the pointwise kernel (:1118-1178) over the node -> code recursion of
 *    src/codegen.rs:283-443. The carrier is the reference's own: leaves, into, combine, identity, project
 *    (src/derive.rs:262-287) over the closed scalar basis (src/scalar.rs:45-69, Expr src/derive.rs:96-118). ── */
#define SANIC_MAX_AXES 6
#define SANIC_MAX_SLOTS 8
enum { SANIC_X_CONST = 1,   /* value */
       SANIC_X_LOAD = 2,    /* arg = operand index: a typed, strided read at the current point */
       SANIC_X_COORD = 3,   /* arg = grid axis, n_axes for the streamed coordinate, n_axes + 2 + j for window coordinate j of a
                               streamed window of several axes, n_axes + 1 for the inner coordinate of a
                               contracted leaf; as a float (Iota / Coordinate) */
       SANIC_X_ITEM = 4,    /* arg = leaf index (into, and project for stream-invariant leaves is not needed: use LOAD) */
       SANIC_X_A = 5, SANIC_X_B = 6,   /* arg = slot of the left / right accumulator (combine) */
       SANIC_X_F = 7,       /* arg = slot of the final accumulator (project) */
       SANIC_X_RESULT = 8,  /* the projected value (epilogue) */
       SANIC_X_GATHER = 9,  /* arg = operand index; pops the index value: reads the operand at round(index) along its gather
                               axis (Gather: round, then a bounds check, src/interp.rs:378-379). An index out of range reads 0
                               and the next sanic_sync fails with SANIC_ERR_INVALID */
       SANIC_X_GATHER_PAD = 10, /* the same read where an index out of range is padding: it reads 0 and is no error (a padded
                               Reindex reads 0.0, src/interp.rs:270-430: padded windows of convolutions and sliding windows) */
       SANIC_X_ADD = 16, SANIC_X_SUB, SANIC_X_MUL, SANIC_X_DIV, SANIC_X_MAX, SANIC_X_MIN,
       SANIC_X_LT,          /* a < b as 1.0 / 0.0 */
       SANIC_X_NEG, SANIC_X_RECIP, SANIC_X_EXP, SANIC_X_LOG, SANIC_X_SQRT, SANIC_X_TANH, SANIC_X_SIN, SANIC_X_COS,
       SANIC_X_WHERE,       /* cond != 0 ? a : b; operands pushed cond, a, b */
       SANIC_X_ROUND };     /* arg = SANIC_BF16 / SANIC_F32: round to a storage width and widen back */
typedef struct { int32_t op; int32_t arg; double value; } sanic_expr_op;   /* one postfix instruction */
typedef struct { int32_t first, count; } sanic_expr;                        /* a slice of the op array */
typedef struct {
    int32_t dtype;                      /* SANIC_F32 / SANIC_BF16 / SANIC_U32 / SANIC_I4 (unsigned nibble q+8, low nibble = even element) */
    int32_t buffer;                     /* which of the buffers bound at launch, 0..15 */
    int64_t offset;                     /* elements */
    int64_t stride[SANIC_MAX_AXES];     /* elements per step of each grid axis; 0 broadcasts */
    int64_t stream_stride;              /* elements per step of the streamed axis */
    int64_t inner_stride;               /* elements per step of a contracted leaf's inner axis */
    int64_t gather_stride;              /* elements per step of the gathered index (SANIC_X_GATHER only) */
    int64_t gather_extent;              /* valid indices are 0 .. gather_extent-1 */
    int64_t stream_sub_stride[3];       /* with stream_dims > 1: elements per step of each axis of the streamed window (then
                                           stream_stride is not read) */
} sanic_operand;
typedef struct {
    int32_t n_axes;                     /* output grid, row-major, last axis fastest */
    int64_t extent[SANIC_MAX_AXES];
    int64_t stream;                     /* streamed extent; 0 = pointwise kernel: out[point] = project */
    int32_t lanes;                      /* 1: one thread per output point; 32: a warp per point (cooperative fold) */
    int32_t warps;                      /* lanes == 32 only: 0 or 1 = one warp per point; 2..8 = a block of that many warps per
                                           point, the chunking below taken over all its threads (B = min(32*warps, n)), warp
                                           partials merged in warp order through shared memory */
    int32_t lane_axis;                  /* lanes == 32 only. 1: the LAST grid axis is spread over the lanes (FoldSched::lane_axis,
                                           src/plan.rs:434-455): a warp owns 32 neighbouring points, each lane its own accumulator; a
                                           contracted leaf that does not read that axis is computed once per warp (inner axis split over
                                           the lanes, butterfly sum); with warps > 1 the streamed axis is split over the warps instead
                                           of over the lanes */
    int32_t interleave;                 /* lanes == 32 only. 0: lane b folds the contiguous chunk [b*n/B, (b+1)*n/B), B = min(32, n),
                                           merged in lane order (run_carrier_split, src/interp.rs:597-640): legal for every carrier.
                                           1: lane b folds s = b, b+32, ...: needs a carrier that merges out of order (src/plan.rs:481-488) */
    int32_t n_operands; const sanic_operand* operands;
    int32_t n_ops; const sanic_expr_op* ops;
    int32_t n_leaves; const sanic_expr* leaves;           /* value of leaf i at (point, s): LOAD / COORD / CONST and the basis */
    const int64_t* leaf_inner;                            /* NULL, or per leaf: an extent R > 1 makes the leaf the sum over r < R of
                                                             its program (operands step by inner_stride; COORD n_axes+1 reads r):
                                                             a contraction computed in the fold body (src/codegen.rs:27-36) */
    int32_t n_slots; const double* identity;
    const sanic_expr* into;                               /* per slot, over ITEM */
    const sanic_expr* combine;                            /* per slot, over A and B; all slots read the old accumulator */
    sanic_expr project;                                   /* over F (and LOAD / COORD at the grid point) */
    sanic_expr epilogue;                                  /* count 0 = none; over RESULT and LOAD / COORD at the grid point */
    sanic_expr store_if;                                  /* count 0 = always; else the point is stored only where this is != 0:
                                                             the in-place form of where(c, x, s) writing s's own buffer, which
                                                             never loads s (src/emit_metal.rs:1118-1178) */
    int32_t out_dtype;                                    /* SANIC_F32 / SANIC_BF16 (RNE) / SANIC_U32 (saturating) */
    int32_t stream_dims;                                  /* 0 or 1: the streamed axis is one axis. 2 or 3: it is the row-major
                                                             flattening of a window of that many axes (a reduce over several
                                                             axes at once: the taps and input channels of a convolution, the
                                                             window of a pooling), extents in stream_extent, product = stream;
                                                             operands step by stream_sub_stride and COORD n_axes + 2 + j reads
                                                             the j-th window coordinate */
    int64_t stream_extent[3];
} sanic_generic_desc;
typedef struct sanic_generic_kernel sanic_generic_kernel;
/* The generated CUDA C text (MetalKernel::msl). ctx may be NULL. *needed receives the size including the terminator. */
int32_t sanic_generic_source(sanic_ctx* ctx, const sanic_generic_desc* d, char* buf, size_t cap, size_t* needed);
/* Renders and compiles for sm_100a without loading: the "does the generated code compile" check; needs no device. ctx may be NULL. */
int32_t sanic_generic_cubin_size(sanic_ctx* ctx, const sanic_generic_desc* d, size_t* bytes);
/* Renders, compiles and loads (MetalDevice::compile, src/metal.rs:160-180; a compile failure is a status, not a panic). */
int32_t sanic_generic_compile(sanic_ctx* ctx, const sanic_generic_desc* d, sanic_generic_kernel** out);
/* out holds one element per grid point at the descriptor's out_dtype. */
int32_t sanic_generic_launch(sanic_ctx* ctx, sanic_generic_kernel* k, const void* const* buffers, int32_t n_buffers, void* out,
                             void* stream);
int32_t sanic_generic_destroy(sanic_generic_kernel* k);
/* A descriptive name of the kernel (kind, grid, streamed extent, schedule, output width): kernel_name of the reference's
 * emitter (src/emit_metal.rs:1340-1370); a debug stage listing prints it. */
const char* sanic_generic_kernel_name(sanic_generic_kernel* k);
/* Kernel dedup across isomorphic stages (src/emit_metal.rs:1281-1330): stages that differ only in their buffers render the
 * same text and are compiled once per process. Counts of texts compiled and of compilations answered from the cache. */
int32_t sanic_generic_cache_stats(int64_t* compiled, int64_t* reused);

/* ── stateful stepping: Graph::compile_for / StepProgram::instantiate / Machine::step
 *    (src/graph.rs:231-356) with capture/replay (src/compile.rs:820-1035, src/metal.rs:634-705) ── */
typedef struct sanic_program sanic_program;
enum { SANIC_STAGE_FUSED = 1, SANIC_STAGE_ELEMENTWISE = 2, SANIC_STAGE_GATHER = 3 };  /* src/partition.rs:44-98 */
enum { SANIC_OP_GEMV = 1, SANIC_OP_DECODE_ATTN = 2, SANIC_OP_ARGMAX = 3, SANIC_OP_RMSNORM = 4, SANIC_OP_EMBED = 5,
       SANIC_OP_ROPE_CACHE = 6, SANIC_OP_ADVANCE = 7, SANIC_OP_GENERIC = 8,
       SANIC_OP_ATTN_FWD = 9,      /* the online-softmax fold over many queries: prefill and plain attention (FUSED) */
       SANIC_OP_GEMM_RMSNORM = 10, /* the deferred-normaliser contraction (FUSED) */
       SANIC_OP_ROPE = 11 };       /* rotate-half RoPE of whole [rows, seq, D] operands, the cut the reference makes in front
                                      of a fold over projected operands (src/partition.rs:1295-1311) (ELEMENTWISE) */
typedef struct {
    int32_t stage_kind;          /* SANIC_STAGE_* */
    int32_t op;                  /* SANIC_OP_* */
    sanic_carrier_desc carrier;  /* for FUSED stages: checked against the op by sanic_emit_select */
    union {
        sanic_gemv_params gemv;
        sanic_decode_params decode;
        struct { const float* x; int32_t rows, n; uint32_t* out; float* scratch; } argmax;
        struct { const float* x; const void* gamma; int32_t rows, n; float eps; void* out; } rmsnorm;
        struct { const void* table; const int32_t* tokens; int32_t batch, hidden, vocab; float* out;
                 const void* scales; int32_t table_dtype /* 0 / SANIC_BF16, or SANIC_I4 with scales */, group; } embed;
        sanic_rope_cache_params rope_cache;
        struct { int32_t* position; } advance;
        struct { sanic_generic_kernel* kernel; const void* buffers[16]; int32_t n_buffers; void* out; } generic;   /* a compiled fallback kernel */
        struct { sanic_attn_params p; int32_t storage; /* SANIC_F32: CUDA-core path; SANIC_BF16: tensor-core path */ } attn;
        sanic_gemm_rmsnorm_params gemm;
        struct { const void* x; void* out; int64_t rows; int32_t seq, head_dim; const float* table; int32_t pos0; } rope;
    } u;
} sanic_stage_desc;
int32_t sanic_program_create(sanic_ctx* ctx, const sanic_stage_desc* stages, int32_t n_stages, sanic_program** out);
int32_t sanic_program_destroy(sanic_program* prog);
int32_t sanic_program_kernel_count(sanic_program* prog);
/* Launch every stage in order on `stream` (Backend::execute, src/compile.rs:101-107). */
int32_t sanic_program_run(sanic_program* prog, void* stream);
/* Freeze the launch list into a CUDA graph (MetalDevice::capture) and replay it
 * (MetalReplay::step_timed): gpu_seconds (optional) is the device time of this replay. */
int32_t sanic_program_capture(sanic_program* prog, void* stream);
/* The same, lowered into one cooperative kernel that walks the stage list with grid-wide barriers instead of
 * kernel boundaries (no counterpart in the reference: Metal has one command buffer per step,
 * src/metal.rs:634-705, but no device-wide barrier inside a dispatch). SANIC_ERR_UNSUPPORTED when a stage
 * has no phase in that kernel (RoPE as its own stage, head_dim 128, an inlined norm at batch > 8). */
int32_t sanic_program_capture_persistent(sanic_program* prog, void* stream);
int32_t sanic_program_step(sanic_program* prog, void* stream, double* gpu_seconds);
/* One step with a device time per stage (MetalDevice::run_kernel_timed, src/metal.rs:431-447). `seconds`
 * receives min(cap, stages) entries and *n_out their count; a program captured in its single-kernel form
 * reports one entry per phase (argmax is two). The step is a real one: state advances. Synchronises `stream`. */
int32_t sanic_program_stage_times(sanic_program* prog, void* stream, double* seconds, int32_t cap, int32_t* n_out);
/* A finer view of one step of a program captured in its single-kernel form (the per-kernel breakdown of the
 * reference's SANIC_DEBUG=4 replay, src/compile.rs:1147-1346, inside one kernel): per phase, seconds from the phase's
 * start to (0) its activations staged in shared memory, (1) its last contraction done, (2) its sums and epilogue done,
 * (3) the grid barrier that ends it released, as block 0 saw them; phases that are not contractions report 0, 0, 0 and
 * their whole time. `out` receives 4 * min(cap, phases) numbers. The step is a real one. Synchronises `stream`. */
int32_t sanic_program_phase_profile(sanic_program* prog, void* stream, double* out, int32_t cap, int32_t* n_out);

/* ── schedules over a buffer table: binding by name on every run, replays with state feedback, machines ──
 *
 * What the reference's emitter hands its runtime is a program whose stages NAME their buffers
 * (MetalProgram{stages[{kernel, inputs, output, ..}], inputs, dtypes, buffers[(name, elements)]},
 * src/emit_metal.rs:1183-1212). A schedule here is the stage list above plus that buffer table and a relocation
 * list: each pointer field of a stage that refers to a table buffer is given as (stage, byte offset of the field
 * inside sanic_stage_desc, buffer index, byte offset into the buffer). Binding fills those fields and nothing else,
 * so binding other buffers never recompiles anything. Every check runs on the host before any CUDA call; a
 * schedule compiled with ctx == NULL checks bindings and feedback without a device and refuses to run. */
enum { SANIC_BUF_INPUT = 1,    /* bound by the caller, by name (InputSpec, src/compile.rs:114-121) */
       SANIC_BUF_SCRATCH = 2 };/* allocated by the runtime, zero-filled: intermediates and outputs (program.buffers) */
typedef struct {
    const char* name;                   /* unique; inputs are bound under this name */
    int32_t kind;                       /* SANIC_BUF_* */
    int32_t dtype;                      /* declared storage: SANIC_F32 / F16 / BF16 / U32 / I4 */
    int32_t rank;
    int64_t shape[SANIC_MAX_AXES];      /* concrete extents (dynamic shapes are refused) */
} sanic_buffer_decl;
typedef struct { int32_t stage; int32_t field_offset; int32_t buffer; int64_t byte_offset; } sanic_reloc;
typedef struct {
    const sanic_stage_desc* stages; int32_t n_stages;   /* pointer fields named by a relocation are filled at bind time */
    const sanic_buffer_decl* buffers; int32_t n_buffers;
    const sanic_reloc* relocs; int32_t n_relocs;
    const int32_t* outputs; int32_t n_outputs;          /* buffer index of every root, in compilation-root order */
    /* roots compiled in place (compile_roots_in_place, src/compile.rs:408; the law is Graph::overwritable_states,
     * src/graph.rs:127-160): root in_place_root[i] writes the buffer of input in_place_input[i] (a buffer index) instead
     * of one of its own */
    const int32_t* in_place_root; const int32_t* in_place_input; int32_t n_in_place;
} sanic_schedule_desc;
/* A bound buffer as the runtime sees one: Buffer::shape() and Buffer::dtype() (src/compile.rs:81-84) plus its address. */
typedef struct { const char* name; const void* dptr; int32_t dtype; int32_t rank; int64_t shape[SANIC_MAX_AXES]; } sanic_binding;
typedef struct { void* dptr; int32_t dtype; int32_t rank; int64_t shape[SANIC_MAX_AXES]; size_t bytes; } sanic_buffer_view;
typedef struct sanic_schedule sanic_schedule;
typedef struct sanic_replay sanic_replay;
/* Backend::prepare (src/compile.rs:94-99): validates the table, every stage's structure (kind, op, carrier family, leaf
 * storage), the relocations, the roots and the in-place pairs. */
int32_t sanic_schedule_compile(sanic_ctx* ctx, const sanic_schedule_desc* desc, sanic_schedule** out);
int32_t sanic_schedule_destroy(sanic_schedule* s);
const char* sanic_schedule_last_error(sanic_schedule* s);   /* also set when the schedule has no context; with s == NULL: why
                                                               this thread's last sanic_schedule_compile failed */
int32_t sanic_schedule_input_count(sanic_schedule* s);      /* Program::input_names (src/compile.rs:138-140) */
const char* sanic_schedule_input_name(sanic_schedule* s, int32_t i);
int32_t sanic_schedule_output_count(sanic_schedule* s);
/* The checks of Program::ordered_bindings (src/compile.rs:190-229), alone: SANIC_ERR_UNKNOWN_INPUT, _DUPLICATE_INPUT,
 * _MISSING_INPUT, _SHAPE, _DTYPE in that order of discovery. */
int32_t sanic_schedule_check_bindings(sanic_schedule* s, const sanic_binding* bindings, int32_t n);
/* Program::try_run / Backend::execute (src/compile.rs:101-107,175-187): bind by name, launch every stage on `stream`,
 * return the roots in order. The views point into storage the schedule owns: valid until its next execute or destroy. */
int32_t sanic_schedule_execute(sanic_schedule* s, const sanic_binding* bindings, int32_t n, void* stream,
                               sanic_buffer_view* outputs, int32_t n_outputs);
/* Program::capture(bindings, feedback) (src/compile.rs:820-960): freeze the step over these bindings. Each feedback pair
 * (root index, input name) must name a real root and a real input of equal shape and storage, each at most once
 * (SANIC_ERR_FEEDBACK otherwise). A pair whose root was compiled in place is ONE buffer; any other pair makes the replay
 * two frozen steps whose buffers trade places (ping-pong). persistent != 0 lowers each step into the single cooperative
 * kernel (sanic_program_capture_persistent). */
int32_t sanic_schedule_capture(sanic_schedule* s, const sanic_binding* bindings, int32_t n, const int32_t* feedback_output,
                               const char* const* feedback_input, int32_t n_feedback, int32_t persistent, void* stream,
                               sanic_replay** out);
int32_t sanic_replay_step(sanic_replay* r, void* stream, double* gpu_seconds);           /* MetalReplay::step_timed */
int32_t sanic_replay_stage_times(sanic_replay* r, void* stream, double* seconds, int32_t cap, int32_t* n_out);
int32_t sanic_replay_phase_profile(sanic_replay* r, void* stream, double* out, int32_t cap, int32_t* n_out);
int32_t sanic_replay_output(sanic_replay* r, int32_t root, sanic_buffer_view* out);       /* MetalReplay::last_outputs */
int32_t sanic_replay_kernel_count(sanic_replay* r);
int32_t sanic_replay_parities(sanic_replay* r);                                           /* 1, or 2 when feedback swaps */
int32_t sanic_replay_destroy(sanic_replay* r);
/* Graph::compile_for + StepProgram::instantiate (src/graph.rs:231-341). A state is an input whose successor is root
 * `root`; its buffer is allocated here, zero-filled, and owned by the machine; the caller binds the other inputs only
 * (binding a state is SANIC_ERR_DUPLICATE_INPUT). A state declared at another width than `boundary_dtype`, the
 * compilation's boundary policy, is refused with SANIC_ERR_UNSUPPORTED unless `pinned` (src/graph.rs:236-245,
 * Graph::output_at :113-125). The machine is a replay: step it with sanic_replay_step. */
typedef struct { const char* input_name; int32_t root; int32_t pinned; } sanic_state_decl;
int32_t sanic_machine_instantiate(sanic_schedule* s, const sanic_state_decl* states, int32_t n_states, int32_t boundary_dtype,
                                  const sanic_binding* bindings, int32_t n, const char* const* output_names,
                                  const int32_t* output_roots, int32_t n_named_outputs, int32_t persistent, void* stream,
                                  sanic_replay** out);
int32_t sanic_machine_output(sanic_replay* m, const char* name, sanic_buffer_view* out);  /* Machine::output (src/graph.rs:343-356) */
/* The buffer state `name` will be read from by the NEXT step (to load a prefilled cache, or to read a state back). */
int32_t sanic_machine_state(sanic_replay* m, const char* name, sanic_buffer_view* out);

/* ── planning facts, the device-level split, measured tuning ──
 * sanic_fitted_specs is the reference's DeviceSpecs (src/cost.rs:33-60: sram_bytes ... mem_latency_s, same meaning) with
 * what this device adds. sanic_specs_b200 is the counterpart of DeviceSpecs::m1_pro (src/cost.rs:93-119): constants fitted
 * from this library's own measured kernels on B200. sanic_specs_measure re-measures the ones a probe can give. */
typedef struct {
    double sram_bytes, regfile_bytes, hbm_bandwidth, peak_flops, launch_overhead, dtype_bytes;
    int32_t compute_dtype, boundary_dtype;      /* DeviceSpecs::compute, Policy::boundary */
    double min_blocks, mem_latency_s;
    /* beyond the reference's fields */
    double hbm_read_bandwidth;                  /* a read-only sweep (folds read, they do not copy) */
    double launch_overhead_empty;               /* measured floor: an empty kernel after an empty kernel in a replayed graph */
    double exp_per_clk_per_sm, sm_clock_hz;     /* the SFU rate that bounds the online-softmax fold at small head_dim */
    double grid_barrier_s;                      /* device-wide barrier inside the single-kernel step */
    double exchange_latency_s, link_bandwidth;  /* cross-device carrier exchange: fixed latency, bytes/s per direction */
    double l2_bytes;
    int32_t sm_count, reserved;
} sanic_fitted_specs;
int32_t sanic_specs_b200(sanic_fitted_specs* out);
int32_t sanic_specs_measure(sanic_ctx* ctx, void* stream, sanic_fitted_specs* out);
/* mergeable_out_of_order (src/plan.rs:478-488): 1 when every slot kind re-associates, so the streamed axis may be split. */
int32_t sanic_mergeable_out_of_order(const sanic_carrier_desc* carrier);
/* The chunking of run_carrier_split (src/interp.rs:603) at any level: part `part` of `parts` owns [lo, hi). */
int32_t sanic_shard_range(int64_t extent, int32_t part, int32_t parts, int64_t* lo, int64_t* hi);
/* FoldSched (src/plan.rs:434-476) with the device-level factor on the streamed axis above the kernel: legal for every
 * carrier sanic_mergeable_out_of_order accepts, the carriers being the exchanged state. sanic_plan_fold prices a fold of
 * `points` outputs in `streams` independent operand streams ((batch, kv head) groups), `bytes_per_step` / `flops_per_step`
 * summed over all streams, for device counts 1, 2, 4, 8 (up to max_devices): roofline with the Little's-law bandwidth
 * floor, launch overhead, and for d > 1 the fixed exchange latency plus (d - 1) carriers over the link. Cheapest wins. */
typedef struct {
    int32_t devices;            /* parts of the streamed axis, one per device (1 = no device-level split) */
    int32_t ctas;               /* resident CTAs per device the axis is cut over */
    int32_t warps, lanes;       /* FoldSched::sgs and the lane width inside a CTA */
    double seconds, hbm_seconds, flop_seconds, launch_seconds, exchange_seconds;
} sanic_fold_plan;
int32_t sanic_plan_fold(const sanic_fitted_specs* specs, const sanic_carrier_desc* carrier, int64_t points, int64_t streams,
                        int64_t stream_extent, double bytes_per_step, double flops_per_step, int32_t carrier_floats_per_point,
                        int32_t max_devices, sanic_fold_plan* out);
/* In-context timing of schedule candidates (the reference's SANIC_TUNE path, src/compile.rs:1348-1630) for the decode
 * fold, on the caller's own buffers: candidates[i] > 0 = that many fixed chunks per (batch, kv head), 0 = the stream-K
 * form. p->n_splits must be the largest slot count among them (it sizes p->partials). seconds (optional) receives the best
 * of `repeats` timed launches per candidate, *best_index the fastest. */
int32_t sanic_tune_decode(sanic_ctx* ctx, const sanic_decode_params* p, const int32_t* candidates, int32_t n, int32_t repeats,
                          void* stream, int32_t* best_index, double* seconds);

/* ── multi-device split-KV: each device folds its slice of the key axis, the carriers are
 *    exchanged and merged with the derived combine (src/interp.rs:538-554) ── */
int32_t sanic_nccl_unique_id(uint8_t out_id[128]);
int32_t sanic_nccl_init(sanic_ctx* ctx, int32_t rank, int32_t nranks, const uint8_t id[128]);
int32_t sanic_nccl_shutdown(sanic_ctx* ctx);
/* Host-side bounded wait for work on `stream` that includes a collective: polls the stream and ncclCommGetAsyncError.
 * When `timeout_ms` passes with the stream still busy (a rank never joined: such a collective cannot be waited out on the
 * device) or the communicator reports an error, the communicator is aborted and dropped from the context and the call
 * fails with SANIC_ERR_TIMEOUT / SANIC_ERR_NCCL. Without a communicator, or with timeout_ms <= 0, this is sanic_sync. */
int32_t sanic_nccl_wait(sanic_ctx* ctx, void* stream, int32_t timeout_ms);
/* Runs the local split-KV fold (p->carrier_out must be set, p->out ignored), all-gathers the
 * [rows, 2+D] carriers into `gathered` [nranks, rows, 2+D] and merges them into `out` on every rank. */
int32_t sanic_splitkv_decode_step(sanic_ctx* ctx, const sanic_decode_params* p, float* gathered, void* out,
                                  int32_t out_dtype, void* stream);

/* The same step with the exchange and the merge in one kernel over peer memory instead of NCCL: every device
 * stores its accumulators into each peer's exchange buffer over NVLink, publishes a flag, waits (bounded) for the
 * others' flags and merges in rank order. The reference has no multi-device path; this is the device-level split
 * of src/interp.rs:597-640 with shared memory between devices as the exchange medium.
 * Set-up: every rank allocates sanic_peer_exchange_bytes() with sanic_alloc, zero-fills it, exports it with
 * sanic_ipc_export, sends the 64 bytes to the other ranks by any side channel, and opens theirs with
 * sanic_ipc_open; buffers[rank] is the local allocation itself. All ranks must have zero-filled before the first
 * step (host barrier). `epoch` starts at 1 and increases by 1 every step on every rank. */
typedef struct {
    int32_t rank, nranks;        /* 1..8 */
    void* buffers[8];            /* every rank's exchange buffer as mapped in this process */
    uint32_t epoch;
    uint32_t spin_limit;         /* polls of a peer's flag before the wait gives up with SANIC_ERR_TIMEOUT (code 41 + rank);
                                    0 = the default, about one second. Ranks are assumed to launch their steps within that
                                    skew of each other; a serving loop with long host-side gaps raises it or runs a host
                                    barrier first */
} sanic_peer_exchange;
size_t sanic_peer_exchange_bytes(int32_t rows /* batch * q_heads */, int32_t head_dim, int32_t nranks);
int32_t sanic_ipc_export(sanic_ctx* ctx, const void* dptr, uint8_t handle_out[64]);
int32_t sanic_ipc_open(sanic_ctx* ctx, const uint8_t handle[64], void** dptr_out);
int32_t sanic_ipc_close(sanic_ctx* ctx, void* dptr);
int32_t sanic_splitkv_decode_step_peer(sanic_ctx* ctx, const sanic_decode_params* p, const sanic_peer_exchange* x, void* out,
                                       int32_t out_dtype, void* stream);

/* The multi-device step as ONE launch: the stream-K fold above whose stage 2, per (batch, kv head) group, stores the
 * group's merged accumulators into every device's exchange buffer, publishes a per-group flag, and, after the CTA has
 * finished its own range, waits (bounded; status 41 + rank on expiry) for the other devices' flags of that group, merges
 * in rank order and projects into `out`. No second kernel, no collective. Buffers: sanic_peer_exchange_bytes_fused()
 * bytes each, zero-filled, exchanged as for sanic_splitkv_decode_step_peer; p->out and p->carrier_out are not needed. */
size_t sanic_peer_exchange_bytes_fused(int32_t rows /* batch * q_heads */, int32_t head_dim, int32_t nranks, int32_t groups /* batch * kv_heads */);
int32_t sanic_splitkv_decode_step_fused(sanic_ctx* ctx, const sanic_decode_params* p, const sanic_peer_exchange* x, void* out,
                                        int32_t out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SANIC_B200_H */
