// Multi-device split-KV decode with the exchange and the merge in ONE kernel over peer memory.
//
// After its local fold (attn_decode.cu) every device holds one raw (m, l, o) accumulator per (batch, query
// head): 66,560 bytes for 4 x 32 heads at head_dim 128. The NCCL form (nccl_merge.cu) all-gathers them and
// then launches the merge. Here each device's kernel stores its accumulators straight into every peer's
// exchange buffer over NVLink (plain peer stores through an IPC mapping), publishes one flag per peer with a
// system-scope release, waits (bounded) for the other devices' flags in its own buffer, and merges the
// accumulators left to right in rank order with the derived combine (reference src/derive.rs:1700-1713;
// rank order is chunk order: stage 2 of run_carrier_split, src/interp.rs:597-640). One launch instead of a
// collective plus a kernel; the exchange is latency-bound, so that is what it costs.
//
// Exchange buffer, identical on every device (sanic_peer_exchange_bytes):
//   flags [2 parities][16] u32   epoch of the last accumulator set that rank q has fully stored here
//   data  [2 parities][nranks][rows][2 + D] f32
// Two parities: a fast device may store step e+1 while a slow one still merges step e; it cannot reach step
// e+2 before the slow one has published its step e+1 flag, i.e. finished reading step e.
//
// Plain peer stores and loads only. Every wait is bounded and reports through the status word.
#include <cstring>

#include "common.cuh"

namespace {
using namespace sanic;

constexpr int MAX_RANKS = 8;
constexpr int FLAG_WORDS = 2 * 16;
constexpr unsigned PEER_SPIN_LIMIT = 1u << 21;     // about a second of system-scope polls

struct Peers { float* buf[MAX_RANKS]; };

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256) peer_push_merge_kernel(const float* __restrict__ local, int rows, int D, int rank, int nranks,
                                                            Peers peers, unsigned epoch, unsigned spin_limit, int* ticket, void* out,
                                                            int out_dtype, int* err) {
    const int W = D + 2;
    const int parity = epoch & 1;
    const size_t set_floats = (size_t)rows * W;                       // one rank's accumulators
    const size_t data_off = FLAG_WORDS + (size_t)parity * nranks * set_floats;
    griddep_wait();                                                   // the local fold wrote `local`
    // ── push: this device's accumulators into slot `rank` of every device's buffer (its own included) ──
    const int n4 = (int)(set_floats / 4);                             // rows * (D + 2) is a multiple of 4 for even D
    for (int q = 0; q < nranks; ++q) {
        float4* dst = (float4*)(peers.buf[q] + data_off + (size_t)rank * set_floats);
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = __ldcg((const float4*)local + i);
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
        s_last = (atomicAdd(ticket, 1) == (int)gridDim.x - 1);
        if (s_last) *ticket = 0;
    }
    __syncthreads();
    if (s_last && threadIdx.x < nranks) {
        // every block's stores are fenced and ticketed: tell each device that slot `rank` of this epoch is complete
        __threadfence_system();
        st_release_sys((unsigned*)peers.buf[threadIdx.x] + parity * 16 + rank, epoch);
    }
    // ── wait for every device's flag in the local buffer ──
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        const unsigned* flags = (const unsigned*)peers.buf[rank] + parity * 16;
        int ok = 1;
        for (int q = 0; q < nranks && ok; ++q) {
            unsigned spins = 0;
            while (ld_acquire_sys(flags + q) != epoch) {
                if (++spins > spin_limit) { atomicCAS(err, 0, 41 + q); ok = 0; break; }
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    // ── merge in rank order and project ──
    const float* data = peers.buf[rank] + data_off;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < rows * D; idx += gridDim.x * blockDim.x) {
        const int row = idx / D, d = idx % D;
        const float* pa = data + (size_t)row * W;
        float m = __ldcg(pa), l = __ldcg(pa + 1), ov = __ldcg(pa + 2 + d);
        for (int q = 1; q < nranks; ++q) {
            const float* pb = data + ((size_t)q * rows + row) * W;
            const MloScale sc = mlo_rescale(m, __ldcg(pb));
            l = l * sc.ra + __ldcg(pb + 1) * sc.rb; ov = ov * sc.ra + __ldcg(pb + 2 + d) * sc.rb; m = sc.m;
        }
        const float v = ov / l;
        if (out_dtype == SANIC_BF16) ((uint16_t*)out)[(size_t)row * D + d] = f32_to_bf16_bits(v);
        else ((float*)out)[(size_t)row * D + d] = v;
    }
}
}  // namespace

extern "C" {

size_t sanic_peer_exchange_bytes(int32_t rows, int32_t head_dim, int32_t nranks) {
    if (rows <= 0 || head_dim <= 0 || nranks <= 0) return 0;
    return ((size_t)FLAG_WORDS + 2 * (size_t)nranks * rows * (head_dim + 2)) * 4 + 16;   // + one ticket word, padded
}

int32_t sanic_ipc_export(sanic_ctx* ctx, const void* dptr, uint8_t handle_out[64]) {
    if (!ctx || !dptr || !handle_out) return SANIC_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    sanic_set_device(ctx);
    cudaIpcMemHandle_t h;
    SANIC_CUDA_CHECK(ctx, cudaIpcGetMemHandle(&h, const_cast<void*>(dptr)));
    memcpy(handle_out, &h, 64);
    return SANIC_OK;
}

int32_t sanic_ipc_open(sanic_ctx* ctx, const uint8_t handle[64], void** dptr_out) {
    if (!ctx || !handle || !dptr_out) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    SANIC_CUDA_CHECK(ctx, cudaIpcOpenMemHandle(dptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return SANIC_OK;
}

int32_t sanic_ipc_close(sanic_ctx* ctx, void* dptr) {
    if (!ctx || !dptr) return SANIC_ERR_INVALID;
    sanic_set_device(ctx);
    SANIC_CUDA_CHECK(ctx, cudaIpcCloseMemHandle(dptr));
    return SANIC_OK;
}

int32_t sanic_splitkv_decode_step_peer(sanic_ctx* ctx, const sanic_decode_params* p, const sanic_peer_exchange* x, void* out,
                                       int32_t out_dtype, void* stream) {
    if (!ctx || !p || !x) return SANIC_ERR_INVALID;
    SANIC_REQUIRE(ctx, p->carrier_out && out, "splitkv_decode_step_peer: carrier_out and out are required");
    SANIC_REQUIRE(ctx, x->nranks >= 1 && x->nranks <= MAX_RANKS && x->rank >= 0 && x->rank < x->nranks,
                  "splitkv_decode_step_peer: 1..8 ranks");
    SANIC_REQUIRE(ctx, x->epoch != 0, "splitkv_decode_step_peer: epochs start at 1 (the buffers start zeroed)");
    SANIC_REQUIRE(ctx, ((size_t)p->batch * p->q_heads * (p->head_dim + 2)) % 4 == 0,
                  "splitkv_decode_step_peer: batch * q_heads * (head_dim + 2) must be a multiple of 4");
    SANIC_REQUIRE(ctx, out_dtype == SANIC_BF16 || out_dtype == SANIC_F32, "splitkv_decode_step_peer: bad out dtype");
    Peers peers{};
    for (int q = 0; q < x->nranks; ++q) {
        SANIC_REQUIRE(ctx, x->buffers[q] && ((uintptr_t)x->buffers[q] % 16) == 0, "splitkv_decode_step_peer: missing or misaligned exchange buffer");
        peers.buf[q] = (float*)x->buffers[q];
    }
    sanic_decode_params local = *p;
    local.out = nullptr;  // the local projection is meaningless before the cross-device merge
    int32_t rc = sanic_attn_decode_splitkv(ctx, &local, stream);
    if (rc != SANIC_OK) return rc;
    const int rows = p->batch * p->q_heads;
    const size_t set_floats = (size_t)rows * (p->head_dim + 2);
    int* ticket = (int*)((float*)x->buffers[x->rank] + FLAG_WORDS + 2 * (size_t)x->nranks * set_floats);
    // few blocks, all resident: a block that waits for remote flags must never keep the block that publishes the
    // local one from being scheduled
    int grid = (int)((set_floats / 4 + 255) / 256);
    if (grid > 32) grid = 32;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_pdl(peer_push_merge_kernel, dim3(grid), dim3(256), (size_t)0, (cudaStream_t)stream,
                               (const float*)p->carrier_out, rows, (int)p->head_dim, (int)x->rank, (int)x->nranks, peers,
                               (unsigned)x->epoch, (unsigned)(x->spin_limit ? x->spin_limit : PEER_SPIN_LIMIT), ticket, out, (int)out_dtype,
                               ctx->status_dev);
    if (e != cudaSuccess) return sanic_fail(ctx, SANIC_ERR_CUDA, std::string("splitkv_decode_step_peer: ") + cudaGetErrorString(e));
    return SANIC_OK;
}

}  // extern "C"
