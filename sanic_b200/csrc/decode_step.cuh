// One decode step as ONE persistent kernel: the stage list of a program becomes a phase table that a
// co-resident grid walks, with a grid-wide barrier between phases instead of a kernel boundary.
#pragma once
#include <vector>

#include "common.cuh"

namespace sanic {
namespace step {

struct Plan;

// Builds the phase table for `stages`. Returns SANIC_ERR_UNSUPPORTED (and leaves *out null) when the list
// holds a stage the persistent kernel does not implement; the caller then keeps its launch list.
int32_t build(sanic_ctx* ctx, const std::vector<sanic_stage_desc>& stages, Plan** out);
// Enqueues one step: a 4-byte clear of the barrier word, then the cooperative launch.
int32_t launch(sanic_ctx* ctx, Plan* plan, cudaStream_t stream);
int phases(const Plan* plan);
int32_t phase_times(sanic_ctx* ctx, Plan* plan, double* seconds, int cap);
// Four numbers per phase of the last completed step: staged / contracted / finished / barrier released, in seconds from the phase's start.
int32_t phase_profile(sanic_ctx* ctx, Plan* plan, double* out, int cap);
void destroy(Plan* plan);
// One contraction stage fed through a shared-memory ring by bulk copies (batch > 8): see gemv_ring_kernel.
// SANIC_ERR_UNSUPPORTED when the shape has no ring geometry (no error text is set).
int32_t gemv_ring(sanic_ctx* ctx, const sanic_gemv_params* p, cudaStream_t stream);

}  // namespace step

namespace gemv {
// Whether sanic_gemv serves this contraction with the warp-per-tile int4 kernel (gemv.cu: int4-g64 weights, batch <= 8, one
// matrix of many row tiles, plain store): a program captured in its single-kernel form leaves such a stage, and what
// follows it, to the launch list, because that kernel streams a vocabulary-sized matrix more than twice as fast as the
// step kernel's eight consumer warps do.
bool rows_form_applies(const sanic_ctx* ctx, const sanic_gemv_params& p);
}  // namespace gemv
}  // namespace sanic
