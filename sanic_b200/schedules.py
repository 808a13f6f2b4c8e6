"""Schedules of the one-shot graphs: what `root.compile(&backend)` hands the runtime for attention, the RMSNorm-fused
GEMM and split-KV decode (reference src/compile.rs:87-229 for the boundary; the stage shapes are the ones the reference's
partitioner pins: plain / causal attention is ONE fused stage with three slots that reads only Q, K, V
(src/partition.rs:2491-2513, 3035-3053); RMSNorm with literal eps and 1/n followed by a matmul is ONE stage with two
slots (src/partition.rs:2591-2608); a fold over RoPE'd operands cuts the rotated operands whole in front of it
(src/partition.rs:1295-1311)). Each function returns a ScheduleBuilder whose inputs are bound by name at every run."""
import math

from . import _abi as abi
from .backend import carrier_deferred_norm, carrier_online_softmax
from .schedule import ScheduleBuilder


def attention(batch, q_heads, kv_heads, q_len, kv_len, head_dim, v_dim=None, storage=abi.F32, causal=False, window=0,
              scale=None, rope=False, f64_accumulate=False):
    """softmax(Q K^T * scale + mask) V as one fused stage. Inputs `q` [B,Hq,L,E], `k` [B,Hkv,S,E], `v` [B,Hkv,S,Ev]
    in `storage` (f32: CUDA-core fold; bf16: tensor-core fold); with `rope`, an input `rope_table` [>=max(L,S), E/2, 2]
    f32 and two elementwise stages that rotate q and k into scratch first. Root: `out` [B,Hq,L,Ev]."""
    v_dim = head_dim if v_dim is None else v_dim
    if rope and storage != abi.BF16:
        raise ValueError("the RoPE stage rotates bf16 operands")
    b = ScheduleBuilder()
    b.input("q", storage, (batch, q_heads, q_len, head_dim))
    b.input("k", storage, (batch, kv_heads, kv_len, head_dim))
    b.input("v", storage, (batch, kv_heads, kv_len, v_dim))
    q_name, k_name = "q", "k"
    if rope:
        b.input("rope_table", abi.F32, (max(q_len, kv_len), head_dim // 2, 2))
        for name, heads, seq in (("q", q_heads, q_len), ("k", kv_heads, kv_len)):
            b.scratch(name + ".rotated", storage, (batch, heads, seq, head_dim))
            s = abi.StageDesc()
            s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_ROPE
            r = s.u.rope
            r.rows, r.seq, r.head_dim, r.pos0 = batch * heads, seq, head_dim, 0
            b.stage(s, {"rope.x": name, "rope.out": name + ".rotated", "rope.table": "rope_table"})
        q_name, k_name = "q.rotated", "k.rotated"
    b.scratch("out", storage, (batch, q_heads, q_len, v_dim))
    s = abi.StageDesc()
    s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_ATTN_FWD
    s.carrier = carrier_online_softmax(storage)
    s.u.attn.storage = storage
    p = s.u.attn.p
    p.batch, p.q_heads, p.kv_heads = batch, q_heads, kv_heads
    p.q_len, p.kv_len, p.head_dim, p.v_dim = q_len, kv_len, head_dim, v_dim
    p.causal, p.window = int(causal), int(window)
    p.scale = float(scale if scale is not None else 1.0 / math.sqrt(head_dim))
    p.out_dtype = storage
    p.accum_dtype = abi.F64 if f64_accumulate else abi.F32
    b.stage(s, {"attn.p.q": q_name, "attn.p.k": k_name, "attn.p.v": "v", "attn.p.out": "out"})
    b.root("out")
    return b


def rmsnorm_gemm(M, K, N, w_is_nk=True, eps=1e-5, out_dtype=abi.BF16):
    """y = (x / sqrt(mean(x^2) + eps) * gamma) W as one fused stage. Inputs `x` [M,K], `gamma` [K], `w` [N,K] or [K,N],
    all bf16. Root: `y` [M,N]."""
    b = ScheduleBuilder()
    b.input("x", abi.BF16, (M, K))
    b.input("gamma", abi.BF16, (K,))
    b.input("w", abi.BF16, (N, K) if w_is_nk else (K, N))
    b.scratch("y", out_dtype, (M, N))
    s = abi.StageDesc()
    s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_GEMM_RMSNORM
    s.carrier = carrier_deferred_norm(abi.BF16)
    g = s.u.gemm
    g.M, g.N, g.K, g.w_is_nk, g.eps, g.out_dtype = M, N, K, int(w_is_nk), float(eps), out_dtype
    b.stage(s, {"gemm.x": "x", "gemm.gamma": "gamma", "gemm.w": "w", "gemm.y": "y"})
    b.root("y")
    return b


def splitkv_decode(batch, q_heads, kv_heads, kv_len, head_dim, n_splits, scale=None, window=0):
    """One query token per sequence against `kv_len` keys, folded in `n_splits` contiguous chunks per (batch, kv head)
    and merged with the derived combine (run_carrier_split, src/interp.rs:555-643). Inputs `q` [B,Hq,D], `k`, `v`
    [B,Hkv,S,D] bf16. Root: `out` [B,Hq,D] f32; the partial carriers are a scratch buffer of the schedule."""
    b = ScheduleBuilder()
    b.input("q", abi.BF16, (batch, q_heads, head_dim))
    b.input("k", abi.BF16, (batch, kv_heads, kv_len, head_dim))
    b.input("v", abi.BF16, (batch, kv_heads, kv_len, head_dim))
    # raw (m, l, o) per chunk, then one arrival counter per (batch, q head): the layout sanic_attn_decode_scratch_bytes gives
    b.scratch("partials", abi.F32, (batch * q_heads * (n_splits * (head_dim + 2) + 1),))
    b.scratch("out", abi.F32, (batch, q_heads, head_dim))
    s = abi.StageDesc()
    s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_DECODE_ATTN
    s.carrier = carrier_online_softmax(abi.BF16)
    d = s.u.decode
    d.k_batch_stride, d.k_head_stride, d.k_seq_stride = kv_heads * kv_len * head_dim, kv_len * head_dim, head_dim
    d.v_batch_stride, d.v_head_stride, d.v_row_stride = kv_heads * kv_len * head_dim, kv_len * head_dim, head_dim
    d.v_transposed = 0
    d.batch, d.q_heads, d.kv_heads, d.head_dim, d.kv_len = batch, q_heads, kv_heads, head_dim, kv_len
    d.window, d.n_splits = int(window), int(n_splits)
    d.scale = float(scale if scale is not None else 1.0 / math.sqrt(head_dim))
    d.out_dtype, d.kv_cap = abi.F32, kv_len
    b.stage(s, {"decode.q": "q", "decode.k": "k", "decode.v": "v", "decode.partials": "partials", "decode.out": "out"})
    b.root("out")
    return b
