"""ctypes declarations of include/sanic_b200.h.

The library is required: importing this module raises if libsanic_b200.so has not been
built. There is no CPU fallback behind any of these entry points.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsanic_b200.so")

(OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NCCL, ERR_DTYPE, ERR_NOMEM, ERR_MISSING_INPUT, ERR_UNKNOWN_INPUT,
 ERR_DUPLICATE_INPUT, ERR_SHAPE, ERR_FEEDBACK) = range(13)
BUF_INPUT, BUF_SCRATCH = 1, 2
F32, F16, BF16, U32, I4, F64 = 1, 2, 3, 4, 5, 6
SLOT_PLAIN_ADD, SLOT_PLAIN_MAX, SLOT_PLAIN_MIN, SLOT_EXP_SHIFTED, SLOT_AT_EXTREMUM = 1, 2, 3, 4, 5
KERNEL_NONE, KERNEL_ONLINE_SOFTMAX_FOLD, KERNEL_DEFERRED_NORM_CONTRACTION, KERNEL_PLAIN_CONTRACTION, \
    KERNEL_GROUPED_I4_CONTRACTION, KERNEL_EXTREMUM_INDEX = range(6)
EPI_STORE, EPI_RESIDUAL_ADD, EPI_SILU_MUL, EPI_ROPE_CACHE = 0, 1, 2, 3
STAGE_FUSED, STAGE_ELEMENTWISE, STAGE_GATHER = 1, 2, 3
OP_GEMV, OP_DECODE_ATTN, OP_ARGMAX, OP_RMSNORM, OP_EMBED, OP_ROPE_CACHE, OP_ADVANCE, OP_GENERIC = 1, 2, 3, 4, 5, 6, 7, 8
OP_ATTN_FWD, OP_GEMM_RMSNORM, OP_ROPE = 9, 10, 11
MAX_AXES, MAX_SLOTS = 6, 8
X_CONST, X_LOAD, X_COORD, X_ITEM, X_A, X_B, X_F, X_RESULT, X_GATHER, X_GATHER_PAD = 1, 2, 3, 4, 5, 6, 7, 8, 9, 10
(X_ADD, X_SUB, X_MUL, X_DIV, X_MAX, X_MIN, X_LT, X_NEG, X_RECIP, X_EXP, X_LOG, X_SQRT, X_TANH, X_SIN, X_COS, X_WHERE,
 X_ROUND) = range(16, 33)

vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class DeviceSpecs(C.Structure):
    _fields_ = [("sm_count", i32), ("cc_major", i32), ("cc_minor", i32), ("max_smem_per_block", i32), ("l2_bytes", i32),
                ("warp", i32), ("hbm_bytes", C.c_uint64), ("hbm_gbs_nominal", C.c_double),
                ("bf16_tflops_nominal", C.c_double)]


class CarrierDesc(C.Structure):
    _fields_ = [("n_slots", i32), ("kind", i32 * 4), ("ref", i32 * 4), ("leaf_dtype", i32),
                ("in_body_contraction", i32), ("deferred_div", i32)]


class AttnParams(C.Structure):
    _fields_ = [("q", vp), ("k", vp), ("v", vp), ("out", vp), ("batch", i32), ("q_heads", i32), ("kv_heads", i32),
                ("q_len", i32), ("kv_len", i32), ("head_dim", i32), ("v_dim", i32), ("causal", i32), ("window", i32),
                ("scale", f32), ("mask", vp), ("out_dtype", i32), ("accum_dtype", i32)]


class PeerExchange(C.Structure):
    _fields_ = [("rank", i32), ("nranks", i32), ("buffers", vp * 8), ("epoch", C.c_uint32), ("spin_limit", C.c_uint32)]


class DecodeParams(C.Structure):
    _fields_ = [("q", vp), ("k", vp), ("v", vp),
                ("k_batch_stride", i64), ("k_head_stride", i64), ("k_seq_stride", i64),
                ("v_batch_stride", i64), ("v_head_stride", i64), ("v_row_stride", i64),
                ("v_transposed", i32), ("batch", i32), ("q_heads", i32), ("kv_heads", i32), ("head_dim", i32),
                ("kv_len", i32), ("kv_len_dev", vp), ("window", i32), ("n_splits", i32), ("scale", f32),
                ("partials", vp), ("carrier_out", vp), ("out", vp), ("out_dtype", i32), ("kv_cap", i32)]


class GemmRmsnormParams(C.Structure):
    _fields_ = [("x", vp), ("gamma", vp), ("w", vp), ("y", vp), ("M", i32), ("N", i32), ("K", i32), ("w_is_nk", i32),
                ("eps", f32), ("out_dtype", i32)]


class GemvParams(C.Structure):
    _fields_ = [("x", vp), ("batch", i32), ("K", i32), ("weight_dtype", i32), ("group", i32), ("n_segments", i32),
                ("w", vp * 3), ("scales", vp * 3), ("rows", i32 * 3), ("out", vp * 3), ("out_dtype", i32),
                ("epilogue", i32), ("residual", vp), ("norm_x", vp), ("norm_gamma", vp), ("norm_eps", f32),
                ("rope_table", vp), ("rope_position", vp), ("rope_q_out", vp), ("rope_k_cache", vp), ("rope_v_cache", vp),
                ("rope_q_heads", i32), ("rope_kv_heads", i32), ("rope_head_dim", i32), ("rope_ctx", i32),
                ("nx_out", vp), ("nx_gamma", vp), ("nx_partial", vp), ("ds_partial", vp), ("ds_tiles", i32), ("ds_eps", f32)]


class RopeCacheParams(C.Structure):
    _fields_ = [("q", vp), ("k", vp), ("v", vp), ("q_out", vp), ("k_cache", vp), ("v_cache", vp), ("table", vp),
                ("position", vp), ("batch", i32), ("q_heads", i32), ("kv_heads", i32), ("head_dim", i32), ("ctx", i32)]


class _ArgmaxStage(C.Structure):
    _fields_ = [("x", vp), ("rows", i32), ("n", i32), ("out", vp), ("scratch", vp)]


class _RmsnormStage(C.Structure):
    _fields_ = [("x", vp), ("gamma", vp), ("rows", i32), ("n", i32), ("eps", f32), ("out", vp)]


class _EmbedStage(C.Structure):
    _fields_ = [("table", vp), ("tokens", vp), ("batch", i32), ("hidden", i32), ("vocab", i32), ("out", vp),
                ("scales", vp), ("table_dtype", i32), ("group", i32)]


class _AdvanceStage(C.Structure):
    _fields_ = [("position", vp)]


class _GenericStage(C.Structure):
    _fields_ = [("kernel", vp), ("buffers", vp * 16), ("n_buffers", i32), ("out", vp)]


class _AttnStage(C.Structure):
    _fields_ = [("p", AttnParams), ("storage", i32)]


class _RopeStage(C.Structure):
    _fields_ = [("x", vp), ("out", vp), ("rows", i64), ("seq", i32), ("head_dim", i32), ("table", vp), ("pos0", i32)]


class _StageUnion(C.Union):
    _fields_ = [("gemv", GemvParams), ("decode", DecodeParams), ("argmax", _ArgmaxStage), ("rmsnorm", _RmsnormStage),
                ("embed", _EmbedStage), ("rope_cache", RopeCacheParams), ("advance", _AdvanceStage),
                ("generic", _GenericStage), ("attn", _AttnStage), ("gemm", GemmRmsnormParams), ("rope", _RopeStage)]


class StageDesc(C.Structure):
    _fields_ = [("stage_kind", i32), ("op", i32), ("carrier", CarrierDesc), ("u", _StageUnion)]


class ExprOp(C.Structure):
    _fields_ = [("op", i32), ("arg", i32), ("value", C.c_double)]


class Expr(C.Structure):
    _fields_ = [("first", i32), ("count", i32)]


class Operand(C.Structure):
    _fields_ = [("dtype", i32), ("buffer", i32), ("offset", i64), ("stride", i64 * MAX_AXES), ("stream_stride", i64),
                ("inner_stride", i64), ("gather_stride", i64), ("gather_extent", i64), ("stream_sub_stride", i64 * 3)]


class GenericDesc(C.Structure):
    _fields_ = [("n_axes", i32), ("extent", i64 * MAX_AXES), ("stream", i64), ("lanes", i32), ("warps", i32), ("lane_axis", i32), ("interleave", i32),
                ("n_operands", i32), ("operands", C.POINTER(Operand)), ("n_ops", i32), ("ops", C.POINTER(ExprOp)),
                ("n_leaves", i32), ("leaves", C.POINTER(Expr)), ("leaf_inner", C.POINTER(i64)), ("n_slots", i32), ("identity", C.POINTER(C.c_double)),
                ("into", C.POINTER(Expr)), ("combine", C.POINTER(Expr)), ("project", Expr), ("epilogue", Expr),
                ("store_if", Expr), ("out_dtype", i32), ("stream_dims", i32), ("stream_extent", i64 * 3)]


class BufferDecl(C.Structure):
    _fields_ = [("name", C.c_char_p), ("kind", i32), ("dtype", i32), ("rank", i32), ("shape", i64 * MAX_AXES)]


class Reloc(C.Structure):
    _fields_ = [("stage", i32), ("field_offset", i32), ("buffer", i32), ("byte_offset", i64)]


class ScheduleDesc(C.Structure):
    _fields_ = [("stages", vp), ("n_stages", i32), ("buffers", vp), ("n_buffers", i32), ("relocs", vp), ("n_relocs", i32),
                ("outputs", vp), ("n_outputs", i32), ("in_place_root", vp), ("in_place_input", vp), ("n_in_place", i32)]


class Binding(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dptr", vp), ("dtype", i32), ("rank", i32), ("shape", i64 * MAX_AXES)]


class BufferView(C.Structure):
    _fields_ = [("dptr", vp), ("dtype", i32), ("rank", i32), ("shape", i64 * MAX_AXES), ("bytes", C.c_size_t)]


class StateDecl(C.Structure):
    _fields_ = [("input_name", C.c_char_p), ("root", i32), ("pinned", i32)]


class FittedSpecs(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("sram_bytes", "regfile_bytes", "hbm_bandwidth", "peak_flops", "launch_overhead", "dtype_bytes")] + \
               [("compute_dtype", i32), ("boundary_dtype", i32)] + \
               [(n, C.c_double) for n in ("min_blocks", "mem_latency_s", "hbm_read_bandwidth", "launch_overhead_empty", "exp_per_clk_per_sm",
                                          "sm_clock_hz", "grid_barrier_s", "exchange_latency_s", "link_bandwidth", "l2_bytes")] + \
               [("sm_count", i32), ("reserved", i32)]


class FoldPlan(C.Structure):
    _fields_ = [("devices", i32), ("ctas", i32), ("warps", i32), ("lanes", i32)] + \
               [(n, C.c_double) for n in ("seconds", "hbm_seconds", "flop_seconds", "launch_seconds", "exchange_seconds")]


def dtype_of_torch(dt):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: U32, torch.uint8: I4}[dt]


# name -> (restype, argtypes); every symbol the header declares
PROTOTYPES = {
    "sanic_cuda_open": (i32, [i32, C.POINTER(vp)]),
    "sanic_cuda_close": (i32, [vp]),
    "sanic_last_error": (C.c_char_p, [vp]),
    "sanic_version": (C.c_char_p, []),
    "sanic_specs": (i32, [vp, C.POINTER(DeviceSpecs)]),
    "sanic_probe_sfu": (i32, [vp, i32, i32, i32, vp, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "sanic_probe_stream": (i32, [vp, vp, C.c_size_t, i32, vp, C.POINTER(C.c_double)]),
    "sanic_alloc": (i32, [vp, C.c_size_t, C.POINTER(vp)]),
    "sanic_free": (i32, [vp, vp]),
    "sanic_upload": (i32, [vp, vp, vp, C.c_size_t, vp]),
    "sanic_download": (i32, [vp, vp, vp, C.c_size_t, vp]),
    "sanic_memset": (i32, [vp, vp, i32, C.c_size_t, vp]),
    "sanic_sync": (i32, [vp, vp]),
    "sanic_emit_select": (i32, [C.POINTER(CarrierDesc), C.POINTER(i32)]),
    "sanic_attn_fwd_f32": (i32, [vp, C.POINTER(AttnParams), vp]),
    "sanic_attn_fwd_bf16": (i32, [vp, C.POINTER(AttnParams), vp]),
    "sanic_status_inject": (i32, [vp, i32]),
    "sanic_count_nonfinite": (i32, [vp, vp, C.c_size_t, i32, vp, C.POINTER(C.c_uint32)]),
    "sanic_embed_gather_w4": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]),
    "sanic_attn_decode_splitkv": (i32, [vp, C.POINTER(DecodeParams), vp]),
    "sanic_attn_decode_streamk": (i32, [vp, C.POINTER(DecodeParams), vp]),
    "sanic_attn_decode_streamk_slots": (i32, [vp, i32, i32, i32]),
    "sanic_peer_exchange_bytes_fused": (C.c_size_t, [i32, i32, i32, i32]),
    "sanic_splitkv_decode_step_fused": (i32, [vp, C.POINTER(DecodeParams), C.POINTER(PeerExchange), vp, i32, vp]),
    "sanic_attn_decode_splitkv_static": (i32, [vp, C.POINTER(DecodeParams), vp]),
    "sanic_attn_decode_static_scratch_capacity": (C.c_size_t, []),
    "sanic_attn_decode_scratch_bytes": (C.c_size_t, [i32, i32, i32, i32]),
    "sanic_attn_decode_suggest_splits": (i32, [vp, i32, i32, i32, i64]),
    "sanic_carrier_merge": (i32, [vp, vp, i32, i32, i32, vp, vp, i32, vp]),
    "sanic_gemm_rmsnorm": (i32, [vp, C.POINTER(GemmRmsnormParams), vp]),
    "sanic_attn_fwd_bf16_profile": (i32, [vp, C.POINTER(AttnParams), vp, C.POINTER(C.c_uint64)]),
    "sanic_gemm_rmsnorm_pair_profile": (i32, [vp, C.POINTER(GemmRmsnormParams), vp, C.POINTER(C.c_uint64)]),
    "sanic_gemm_prescale_weights": (i32, [vp, vp, vp, vp, i32, i32, i32, vp]),
    "sanic_gemv": (i32, [vp, C.POINTER(GemvParams), vp]),
    "sanic_argmax": (i32, [vp, vp, i32, i32, vp, vp, vp]),
    "sanic_rmsnorm": (i32, [vp, vp, vp, i32, i32, f32, vp, vp]),
    "sanic_embed_gather": (i32, [vp, vp, vp, i32, i32, i32, vp, vp]),
    "sanic_rope_table": (i32, [vp, C.POINTER(C.c_double), i32, i32, vp, vp]),
    "sanic_rope_bf16": (i32, [vp, vp, vp, i64, i32, i32, vp, i32, vp]),
    "sanic_rope_cache_write": (i32, [vp, C.POINTER(RopeCacheParams), vp]),
    "sanic_advance_position": (i32, [vp, vp, vp]),
    "sanic_round_to_bf16": (i32, [vp, vp, C.c_size_t, vp, vp]),
    "sanic_store_u32_saturating": (i32, [vp, vp, C.c_size_t, vp, vp]),
    "sanic_w4_unpack": (i32, [vp, vp, C.c_size_t, vp, vp]),
    "sanic_generic_source": (i32, [vp, C.POINTER(GenericDesc), C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "sanic_generic_cubin_size": (i32, [vp, C.POINTER(GenericDesc), C.POINTER(C.c_size_t)]),
    "sanic_generic_compile": (i32, [vp, C.POINTER(GenericDesc), C.POINTER(vp)]),
    "sanic_generic_launch": (i32, [vp, vp, C.POINTER(vp), i32, vp, vp]),
    "sanic_generic_destroy": (i32, [vp]),
    "sanic_generic_kernel_name": (C.c_char_p, [vp]),
    "sanic_generic_cache_stats": (i32, [C.POINTER(i64), C.POINTER(i64)]),
    "sanic_program_create": (i32, [vp, C.POINTER(StageDesc), i32, C.POINTER(vp)]),
    "sanic_program_destroy": (i32, [vp]),
    "sanic_program_kernel_count": (i32, [vp]),
    "sanic_program_run": (i32, [vp, vp]),
    "sanic_program_capture": (i32, [vp, vp]),
    "sanic_program_capture_persistent": (i32, [vp, vp]),
    "sanic_program_step": (i32, [vp, vp, C.POINTER(C.c_double)]),
    "sanic_program_stage_times": (i32, [vp, vp, C.POINTER(C.c_double), i32, C.POINTER(i32)]),
    "sanic_schedule_compile": (i32, [vp, C.POINTER(ScheduleDesc), C.POINTER(vp)]),
    "sanic_schedule_destroy": (i32, [vp]),
    "sanic_schedule_last_error": (C.c_char_p, [vp]),
    "sanic_schedule_input_count": (i32, [vp]),
    "sanic_schedule_input_name": (C.c_char_p, [vp, i32]),
    "sanic_schedule_output_count": (i32, [vp]),
    "sanic_schedule_check_bindings": (i32, [vp, C.POINTER(Binding), i32]),
    "sanic_schedule_execute": (i32, [vp, C.POINTER(Binding), i32, vp, C.POINTER(BufferView), i32]),
    "sanic_schedule_capture": (i32, [vp, C.POINTER(Binding), i32, C.POINTER(i32), C.POINTER(C.c_char_p), i32, i32, vp, C.POINTER(vp)]),
    "sanic_replay_step": (i32, [vp, vp, C.POINTER(C.c_double)]),
    "sanic_replay_stage_times": (i32, [vp, vp, C.POINTER(C.c_double), i32, C.POINTER(i32)]),
    "sanic_replay_output": (i32, [vp, i32, C.POINTER(BufferView)]),
    "sanic_replay_kernel_count": (i32, [vp]),
    "sanic_replay_parities": (i32, [vp]),
    "sanic_replay_destroy": (i32, [vp]),
    "sanic_machine_instantiate": (i32, [vp, C.POINTER(StateDecl), i32, i32, C.POINTER(Binding), i32, C.POINTER(C.c_char_p), C.POINTER(i32),
                                        i32, i32, vp, C.POINTER(vp)]),
    "sanic_machine_output": (i32, [vp, C.c_char_p, C.POINTER(BufferView)]),
    "sanic_machine_state": (i32, [vp, C.c_char_p, C.POINTER(BufferView)]),
    "sanic_program_phase_profile": (i32, [vp, vp, C.POINTER(C.c_double), i32, C.POINTER(i32)]),
    "sanic_replay_phase_profile": (i32, [vp, vp, C.POINTER(C.c_double), i32, C.POINTER(i32)]),
    "sanic_specs_b200": (i32, [C.POINTER(FittedSpecs)]),
    "sanic_specs_measure": (i32, [vp, vp, C.POINTER(FittedSpecs)]),
    "sanic_mergeable_out_of_order": (i32, [C.POINTER(CarrierDesc)]),
    "sanic_shard_range": (i32, [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]),
    "sanic_plan_fold": (i32, [C.POINTER(FittedSpecs), C.POINTER(CarrierDesc), i64, i64, i64, C.c_double, C.c_double, i32, i32, C.POINTER(FoldPlan)]),
    "sanic_tune_decode": (i32, [vp, C.POINTER(DecodeParams), C.POINTER(i32), i32, i32, vp, C.POINTER(i32), C.POINTER(C.c_double)]),
    "sanic_nccl_unique_id": (i32, [C.POINTER(C.c_uint8)]),
    "sanic_nccl_init": (i32, [vp, i32, i32, C.POINTER(C.c_uint8)]),
    "sanic_nccl_shutdown": (i32, [vp]),
    "sanic_nccl_wait": (i32, [vp, vp, i32]),
    "sanic_splitkv_decode_step": (i32, [vp, C.POINTER(DecodeParams), vp, vp, i32, vp]),
    "sanic_peer_exchange_bytes": (C.c_size_t, [i32, i32, i32]),
    "sanic_ipc_export": (i32, [vp, vp, C.POINTER(C.c_uint8)]),
    "sanic_ipc_open": (i32, [vp, C.POINTER(C.c_uint8), C.POINTER(vp)]),
    "sanic_ipc_close": (i32, [vp, vp]),
    "sanic_splitkv_decode_step_peer": (i32, [vp, C.POINTER(DecodeParams), C.POINTER(PeerExchange), vp, i32, vp]),
}

_lib = None


def load():
    """Load libsanic_b200.so and declare every prototype. Raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sanic_b200.build`. "
            "sanic_b200 has no CPU fallback and cannot run without its CUDA library.")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
