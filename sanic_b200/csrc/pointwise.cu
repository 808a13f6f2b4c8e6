// Pointwise, gather and extremum-index stages of a decode step, plus the typed
// load/store helpers exposed for bit-exactness tests. These are the K3/K4 rows of the
// reference emitter (src/emit_metal.rs:123-232, 1118-1178 in the reference project).
#include <vector>

#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"

namespace {
using namespace sanic;

// xn = bf16((x * g) / sqrt(sum(x^2) * (1/n) + eps)); one CTA per row, fixed summation order.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* x, const uint16_t* gamma, int n, float eps,
                                                      uint16_t* out) {
    __shared__ float wsum[8];
    __shared__ float s_den;
    griddep_launch();
    griddep_wait();
    const float* xr = x + (size_t)blockIdx.x * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(xr[i], xr[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.0f;
        for (int w = 0; w < 8; ++w) tot += wsum[w];
        s_den = sqrtf(tot * (1.0f / (float)n) + eps);
    }
    __syncthreads();
    float den = s_den;
    for (int i = threadIdx.x; i < n; i += 256)
        out[(size_t)blockIdx.x * n + i] = f32_to_bf16_bits((xr[i] * bf16_to_f32(gamma[i])) / den);
}

__global__ void embed_gather_kernel(const uint16_t* table, const int32_t* tokens, int hidden, int vocab, float* out) {
    griddep_launch();
    griddep_wait();
    int b = blockIdx.x;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // the host validates; never read out of bounds
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[(size_t)b * hidden + i] = bf16_to_f32(table[(size_t)tok * hidden + i]);
}

// The same gather from an int4 group-quantised table: out[b, i] = (nibble - 8) * scale[tok, i / group], the widened
// value an I4 input means (unsigned q + 8 nibbles, low nibble = even element; exact in f32: 4 bits times 8 bits).
__global__ void embed_gather_w4_kernel(const uint8_t* table, const uint16_t* scales, const int32_t* tokens, int hidden, int vocab,
                                       int group, float* out) {
    griddep_launch();
    griddep_wait();
    int b = blockIdx.x;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint8_t* row = table + (size_t)tok * (hidden / 2);
    const uint16_t* srow = scales + (size_t)tok * (hidden / group);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const int nib = (row[i >> 1] >> ((i & 1) * 4)) & 0xF;
        out[(size_t)b * hidden + i] = (float)(nib - 8) * bf16_to_f32(srow[i / group]);
    }
}

// Non-finite values of a buffer, counted (the reference's SANIC_NANSCAN pass, src/compile.rs:1261-1275).
__global__ void count_nonfinite_kernel(const void* p, size_t n, int dtype, unsigned* count) {
    unsigned local = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v;
        if (dtype == SANIC_F32) v = ((const float*)p)[i];
        else if (dtype == SANIC_BF16) v = bf16_to_f32(((const uint16_t*)p)[i]);
        else v = __half2float(((const __half*)p)[i]);
        if (!(fabsf(v) <= 3.4028234664e38f)) ++local;      // NaN and +-inf both fail the comparison
    }
    local = __reduce_add_sync(0xffffffffu, local);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(count, local);
}

__global__ void rope_table_kernel(const double* inv_freq, int n_freq, int n_pos, float* table) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_freq * n_pos) return;
    int pos = idx / n_freq, f = idx % n_freq;
    double s, c;
    sincos((double)pos * inv_freq[f], &s, &c);
    table[2 * (size_t)idx] = (float)c;
    table[2 * (size_t)idx + 1] = (float)s;
}

// out[p=0,f] = x0*cos - x1*sin ; out[p=1,f] = x1*cos + x0*sin  (pair-major split of head_dim).
// One thread rotates 8 consecutive frequencies of one position for ROPE_ROWS rows (batch x head) in turn: the 64 bytes of
// (cos, sin) it needs are read once and kept in registers, where a thread per row read them again for every row (twice the
// bytes of the data itself, all from L2); per row two 16-byte loads and two 16-byte stores, all rows' loads issued first.
constexpr int ROPE_ROWS = 8;
__global__ void rope_bf16_kernel(const uint16_t* x, uint16_t* out, long long rows, int seq, int D,
                                 const float* __restrict__ table, int pos0) {
    const int F = D / 2, FV = F / 8;
    const long long per_row = (long long)seq * FV;
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long groups = (rows + ROPE_ROWS - 1) / ROPE_ROWS;
    if (idx >= groups * per_row) return;
    const long long g = idx / per_row, sf = idx % per_row;
    const int f = (int)(sf % FV) * 8, s = (int)(sf / FV);
    const float4* cs = (const float4*)(table + 2 * ((size_t)(pos0 + s) * F + f));
    float4 t[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) t[i] = __ldg(cs + i);   // (cos, sin) of frequencies f+2i and f+2i+1
    const long long r0 = g * ROPE_ROWS;
    uint4 a[ROPE_ROWS], b[ROPE_ROWS];
#pragma unroll
    for (int r = 0; r < ROPE_ROWS; ++r) {
        if (r0 + r < rows) {
            const size_t base = ((size_t)(r0 + r) * seq + s) * D;
            a[r] = ldg_stream16((const uint4*)(x + base + f));
            b[r] = ldg_stream16((const uint4*)(x + base + F + f));
        }
    }
#pragma unroll
    for (int r = 0; r < ROPE_ROWS; ++r) {
        if (r0 + r < rows) {
            const size_t base = ((size_t)(r0 + r) * seq + s) * D;
            const uint32_t av[4] = {a[r].x, a[r].y, a[r].z, a[r].w}, bv[4] = {b[r].x, b[r].y, b[r].z, b[r].w};
            uint32_t oa[4], ob[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float x0 = bf16lo(av[i]), x1 = bf16lo(bv[i]), y0 = bf16hi(av[i]), y1 = bf16hi(bv[i]);
                oa[i] = pack_bf16x2(x0 * t[i].x + (-x1) * t[i].y, y0 * t[i].z + (-y1) * t[i].w);
                ob[i] = pack_bf16x2(x1 * t[i].x + x0 * t[i].y, y1 * t[i].z + y0 * t[i].w);
            }
            *(uint4*)(out + base + f) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
            *(uint4*)(out + base + F + f) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        }
    }
}
__global__ void rope_bf16_scalar_kernel(const uint16_t* x, uint16_t* out, long long rows, int seq, int D,
                                        const float* table, int pos0) {
    const int F = D / 2;
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = rows * seq * F;
    if (idx >= total) return;
    int f = (int)(idx % F);
    long long rs = idx / F;
    int s = (int)(rs % seq);
    const float* cs = table + 2 * ((size_t)(pos0 + s) * F + f);
    float c = cs[0], sn = cs[1];
    size_t base = (size_t)rs * D;
    float x0 = bf16_to_f32(x[base + f]), x1 = bf16_to_f32(x[base + F + f]);
    out[base + f] = f32_to_bf16_bits(x0 * c + (-x1) * sn);
    out[base + F + f] = f32_to_bf16_bits(x1 * c + x0 * sn);
}

__global__ void rope_cache_write_kernel(sanic_rope_cache_params p) {
    griddep_launch();
    griddep_wait();
    const int D = p.head_dim, F = D / 2;
    const int heads = p.q_heads + 2 * p.kv_heads;
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.batch * heads * F) return;
    int f = idx % F;
    int h = (idx / F) % heads;
    int b = idx / (F * heads);
    int pos = *p.position;
    if (pos < 0 || pos >= p.ctx) return;
    const float* cs = p.table + 2 * ((size_t)pos * F + f);
    float c = cs[0], sn = cs[1];
    if (h < p.q_heads) {
        const float* q = p.q + ((size_t)b * p.q_heads + h) * D;
        float x0 = q[f], x1 = q[F + f];
        uint16_t* o = (uint16_t*)p.q_out + ((size_t)b * p.q_heads + h) * D;
        o[f] = f32_to_bf16_bits(x0 * c + (-x1) * sn);
        o[F + f] = f32_to_bf16_bits(x1 * c + x0 * sn);
    } else if (h < p.q_heads + p.kv_heads) {
        int hk = h - p.q_heads;
        const float* k = p.k + ((size_t)b * p.kv_heads + hk) * D;
        float x0 = k[f], x1 = k[F + f];
        // in-place where(coord == pos, current, cache): only the written row is touched
        uint16_t* o = (uint16_t*)p.k_cache + (((size_t)b * p.kv_heads + hk) * p.ctx + pos) * D;
        o[f] = f32_to_bf16_bits(x0 * c + (-x1) * sn);
        o[F + f] = f32_to_bf16_bits(x1 * c + x0 * sn);
    } else {
        int hk = h - p.q_heads - p.kv_heads;
        const float* v = p.v + ((size_t)b * p.kv_heads + hk) * D;
        uint16_t* o = (uint16_t*)p.v_cache + ((size_t)b * p.kv_heads + hk) * D * (size_t)p.ctx;
        o[(size_t)f * p.ctx + pos] = f32_to_bf16_bits(v[f]);
        o[(size_t)(F + f) * p.ctx + pos] = f32_to_bf16_bits(v[F + f]);
    }
}

__global__ void advance_kernel(int32_t* position) {
    griddep_wait();
    *position += 1;
}

// Extremal-key payload fold: state (max value, first index). Merge: larger key wins, equal
// keys keep the smaller index (reference src/derive.rs:1714-1735). Symmetric, so any tree works.
__device__ __forceinline__ void amax_merge(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}
constexpr int AMAX_CHUNKS = 128;
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* x, int n, float* scratch) {
    griddep_launch();
    griddep_wait();
    int row = blockIdx.y, chunk = blockIdx.x;
    int lo = (int)(((long long)chunk * n) / AMAX_CHUNKS), hi = (int)(((long long)(chunk + 1) * n) / AMAX_CHUNKS);
    const float* xr = x + (size_t)row * n;
    float v = -INFINITY; int i = 0x7FFFFFFF;
    for (int j = lo + threadIdx.x; j < hi; j += 256) amax_merge(v, i, xr[j], j);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float v2 = __shfl_xor_sync(0xffffffffu, v, o); int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        amax_merge(v, i, v2, i2);
    }
    __shared__ float sv[8]; __shared__ int si[8];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) amax_merge(v, i, sv[w], si[w]);
        scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2] = v;
        scratch[((size_t)row * AMAX_CHUNKS + chunk) * 2 + 1] = __int_as_float(i);
    }
}
__global__ void __launch_bounds__(128) argmax_final_kernel(const float* scratch, uint32_t* out) {
    griddep_launch();
    griddep_wait();
    int row = blockIdx.x;
    float v = scratch[((size_t)row * AMAX_CHUNKS + threadIdx.x) * 2];
    int i = __float_as_int(scratch[((size_t)row * AMAX_CHUNKS + threadIdx.x) * 2 + 1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float v2 = __shfl_xor_sync(0xffffffffu, v, o); int i2 = __shfl_xor_sync(0xffffffffu, i, o);
        amax_merge(v, i, v2, i2);
    }
    __shared__ float sv[4]; __shared__ int si[4];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 4; ++w) amax_merge(v, i, sv[w], si[w]);
        // the +inf identity of an empty fold saturates to u32::MAX
        out[row] = (i == 0x7FFFFFFF) ? 0xFFFFFFFFu : (uint32_t)i;
    }
}

__global__ void round_bf16_kernel(const float* x, size_t n, uint16_t* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_bf16_bits(x[i]);
}
__global__ void store_u32_kernel(const float* x, size_t n, uint32_t* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_u32_sat(x[i]);
}
__global__ void w4_unpack_kernel(const uint8_t* packed, size_t n, float* out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (float)(int)((packed[i >> 1] >> ((i & 1) * 4)) & 0xF) - 8.0f;
}
}  // namespace

extern "C" {

int32_t sanic_rmsnorm(sanic_ctx* ctx, const float* x, const void* gamma, int32_t rows, int32_t n, float eps, void* out,
                      void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, x && gamma && out && rows > 0 && n > 0, "rmsnorm: bad arguments");
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, launch_pdl(rmsnorm_kernel, dim3(rows), dim3(256), 0, (cudaStream_t)stream, x, (const uint16_t*)gamma, n, eps, (uint16_t*)out));
    return SANIC_OK;
}

int32_t sanic_embed_gather(sanic_ctx* ctx, const void* table, const int32_t* tokens, int32_t batch, int32_t hidden,
                           int32_t vocab, float* out, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, table && tokens && out && batch > 0 && hidden > 0 && vocab > 0, "embed_gather: bad arguments");
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, launch_pdl(embed_gather_kernel, dim3(batch), dim3(256), 0, (cudaStream_t)stream, (const uint16_t*)table, tokens, hidden, vocab, out));
    return SANIC_OK;
}

int32_t sanic_count_nonfinite(sanic_ctx* ctx, const void* dptr, size_t n, int32_t dtype, void* stream, uint32_t* count) {
    if (!ctx || !dptr || !count) return SANIC_ERR_INVALID;
    if (dtype != SANIC_F32 && dtype != SANIC_BF16 && dtype != SANIC_F16) return sanic_fail(ctx, SANIC_ERR_DTYPE, "count_nonfinite: f32, bf16 or f16");
    sanic_set_device(ctx);
    unsigned* d = nullptr;
    SANIC_CUDA_CHECK(ctx, cudaMalloc(&d, sizeof(unsigned)));
    cudaError_t e = cudaMemsetAsync(d, 0, sizeof(unsigned), (cudaStream_t)stream);
    if (e == cudaSuccess && n) {
        const int blocks = (int)std::min<size_t>((n + 255) / 256, 1184);
        count_nonfinite_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(dptr, n, dtype, d);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(count, d, sizeof(unsigned), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(d);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("count_nonfinite: ") + cudaGetErrorString(e));
    return SANIC_OK;
}

int32_t sanic_embed_gather_w4(sanic_ctx* ctx, const void* table, const void* scales, const int32_t* tokens, int32_t batch,
                              int32_t hidden, int32_t vocab, int32_t group, float* out, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, table && scales && tokens && out && batch > 0 && hidden > 0 && vocab > 0, "embed_gather_w4: bad arguments");
    SANIC_REQUIRE(ctx, group > 0 && group % 2 == 0 && hidden % group == 0, "embed_gather_w4: hidden must be a multiple of the even group size");
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, launch_pdl(embed_gather_w4_kernel, dim3(batch), dim3(256), 0, (cudaStream_t)stream, (const uint8_t*)table,
                                     (const uint16_t*)scales, tokens, hidden, vocab, group, out));
    return SANIC_OK;
}

int32_t sanic_rope_table(sanic_ctx* ctx, const double* inv_freq_host, int32_t n_freq, int32_t n_pos, float* table,
                         void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, inv_freq_host && table && n_freq > 0 && n_pos > 0, "rope_table: bad arguments");
    sanic_set_device(ctx);
    double* d = nullptr;
    SANIC_CUDA_CHECK(ctx, cudaMalloc(&d, sizeof(double) * n_freq));
    cudaError_t e = cudaMemcpyAsync(d, inv_freq_host, sizeof(double) * n_freq, cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e == cudaSuccess) {
        int total = n_freq * n_pos;
        rope_table_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(d, n_freq, n_pos, table);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(d);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("rope_table: ") + cudaGetErrorString(e));
    return SANIC_OK;
}

int32_t sanic_rope_bf16(sanic_ctx* ctx, const void* x, void* out, int64_t rows, int32_t seq, int32_t head_dim,
                        const float* table, int32_t pos0, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, x && out && table && rows > 0 && seq > 0 && head_dim > 0 && head_dim % 2 == 0 && pos0 >= 0,
                  "rope_bf16: bad arguments");
    sanic_set_device(ctx);
    if (head_dim % 16 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        long long total = ((long long)rows + ROPE_ROWS - 1) / ROPE_ROWS * seq * (head_dim / 16);
        rope_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (const uint16_t*)x, (uint16_t*)out, rows, seq, head_dim, table, pos0);
    } else {
        long long total = (long long)rows * seq * (head_dim / 2);
        rope_bf16_scalar_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (const uint16_t*)x, (uint16_t*)out, rows, seq, head_dim, table, pos0);
    }
    SANIC_LAUNCH_CHECK(ctx, "rope_bf16");
    return SANIC_OK;
}

int32_t sanic_rope_cache_write(sanic_ctx* ctx, const sanic_rope_cache_params* p, void* stream) {
    if (!ctx || !p) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->q && p->k && p->v && p->q_out && p->k_cache && p->v_cache && p->table && p->position,
                  "rope_cache_write: null tensor");
    SANIC_REQUIRE(ctx, p->batch > 0 && p->q_heads > 0 && p->kv_heads > 0 && p->head_dim % 2 == 0 && p->ctx > 0,
                  "rope_cache_write: bad shape");
    sanic_set_device(ctx);
    int total = p->batch * (p->q_heads + 2 * p->kv_heads) * (p->head_dim / 2);
    SANIC_CUDA_CHECK(ctx, launch_pdl(rope_cache_write_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, *p));
    return SANIC_OK;
}

int32_t sanic_advance_position(sanic_ctx* ctx, int32_t* position, void* stream) {
    if (!ctx || !position) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, launch_pdl(advance_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, position));
    return SANIC_OK;
}

int32_t sanic_argmax(sanic_ctx* ctx, const float* x, int32_t rows, int32_t n, uint32_t* out_index, float* scratch,
                     void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, x && out_index && scratch && rows > 0 && n > 0, "argmax: bad arguments");
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, launch_pdl(argmax_partial_kernel, dim3(AMAX_CHUNKS, rows), dim3(256), 0, (cudaStream_t)stream, x, n, scratch));
    SANIC_CUDA_CHECK(ctx, launch_pdl(argmax_final_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)stream, (const float*)scratch, out_index));
    return SANIC_OK;
}

int32_t sanic_round_to_bf16(sanic_ctx* ctx, const float* x, size_t n, uint16_t* out_bits, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, x && out_bits, "round_to_bf16: null tensor");
    if (n == 0) return SANIC_OK;
    sanic_set_device(ctx);
    round_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, out_bits);
    SANIC_LAUNCH_CHECK(ctx, "round_to_bf16");
    return SANIC_OK;
}
int32_t sanic_store_u32_saturating(sanic_ctx* ctx, const float* x, size_t n, uint32_t* out, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, x && out, "store_u32: null tensor");
    if (n == 0) return SANIC_OK;
    sanic_set_device(ctx);
    store_u32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, out);
    SANIC_LAUNCH_CHECK(ctx, "store_u32");
    return SANIC_OK;
}
int32_t sanic_w4_unpack(sanic_ctx* ctx, const uint8_t* packed, size_t n_elems, float* out, void* stream) {
    if (!ctx) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, packed && out, "w4_unpack: null tensor");
    if (n_elems == 0) return SANIC_OK;
    sanic_set_device(ctx);
    w4_unpack_kernel<<<(unsigned)((n_elems + 255) / 256), 256, 0, (cudaStream_t)stream>>>(packed, n_elems, out);
    SANIC_LAUNCH_CHECK(ctx, "w4_unpack");
    return SANIC_OK;
}

}  // extern "C"
