#!/usr/bin/env python
"""Benchmark of the hot path: long-context split-KV decode attention (BASELINE.json config 5).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one decode-attention pass over the whole KV cache (batch 4, 32 query heads, 8 KV
heads, head_dim 128, bf16, 1,048,576 keys per sequence, sharded along the sequence over N
GPUs): each GPU folds its slice to (m, l, o) carriers, the carriers are all-gathered over NCCL
and merged with the derived combine. `value` is whole-job algorithmic HBM GB/s (K and V bytes of
all ranks divided by the max-over-ranks device time); total work is fixed as N grows (strong
scaling). Inputs are seeded synthetic N(0,1) tensors; each rank's slice (>= 2 GB) is far larger
than L2, so every step streams from HBM.

Extra objects on the JSON line: `roofline` (dominant kernel, live CUDA-event timing),
`cpu_baseline` (the CPU oracle timed on a bounded sample), `e2e` (host q in, host output out),
`clocks`, `gpu_launches`, and at N=1 a `suite` with the other single-GPU configurations.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, HQ, HKV, D = 4, 32, 8, 128
L_FULL = 1 << 20
METRIC = "split-KV decode attention HBM throughput (B4 Hq32 Hkv8 D128 bf16, 1,048,576 keys/sequence)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        top = mhz[len(mhz) // 2:] if mhz else []     # samples under load: the upper half
        return {"sm_mhz": (top[len(top) // 2] if top else None), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ───────────────────────── CPU reference arm / cpu_baseline ─────────────────────────
def cpu_sample(l_sample: int, repeats: int = 1, seed: int = 1234):
    """The oracle (a restatement of the reference's dense f64 interpreter path) on a bounded sample:
    all 4x32 heads, `l_sample` keys per sequence. Returns (GB/s of bf16 K+V bytes, seconds, threads)."""
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.default_rng(seed)
    q = orc.round_to(orc.DT_BF16, rng.standard_normal((B, HQ, 1, D)))
    k = orc.round_to(orc.DT_BF16, rng.standard_normal((B, HKV, l_sample, D)))
    v = orc.round_to(orc.DT_BF16, rng.standard_normal((B, HKV, l_sample, D)))
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.sdpa(q, k, v, enable_gqa=True)
        best = min(best, time.perf_counter() - t0)
    nbytes = 2 * B * HKV * l_sample * D * 2
    return nbytes / best / 1e9, best, orc.num_threads()


def run_reference(args):
    """Reference arm: the CPU interpreter path on the box's host cores. The reference is Rust and
    cannot be built here, so this times the oracle port with every host thread OpenMP gives it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    l_sample = args.cpu_sample_keys
    times = []
    for i in range(args.warmup + args.steps):
        gbs, sec, threads = cpu_sample(l_sample, 1, seed=1234 + i)
        if i >= args.warmup:
            times.append(sec)
    sec = sum(times) / len(times)
    nbytes = 2 * B * HKV * l_sample * D * 2
    val = nbytes / sec / 1e9
    sample = f"{l_sample} of {L_FULL} keys per sequence, all {B}x{HQ} heads, dense f64, {threads} OpenMP threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "split-KV decode attention, CPU interpreter path, bounded sample", "sample": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_suite():
    """The reference's CPU path (the dense f64 interpreter, restated by the oracle) timed beside configs 1-4 on bounded
    sub-shapes, with every OpenMP thread and with one (the reference's interpreter is single-threaded)."""
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.default_rng(5)
    threads = orc.num_threads()
    out = {"threads": threads}

    def both(fn):
        t0 = time.perf_counter(); fn(); many = time.perf_counter() - t0
        orc.set_num_threads(1)
        t0 = time.perf_counter(); fn(); one = time.perf_counter() - t0
        orc.set_num_threads(threads)
        return many, one
    # config 1 whole: 67.1 MFLOP
    q, k, v = rng.standard_normal((256, 64)), rng.standard_normal((1024, 64)), rng.standard_normal((1024, 64))
    many, one = both(lambda: orc.sdpa(q, k, v, scale=0.125))
    out["c1"] = {"sample": "the whole configuration", "us": many * 1e6, "us_single_thread": one * 1e6}
    # config 2: 32 of the 4096 rows against the whole W (1/128 of the FLOPs)
    x, g, w = rng.standard_normal((32, 2048)), rng.standard_normal(2048), rng.standard_normal((2048, 8192))
    many, one = both(lambda: orc.rmsnorm_gemm(x, g, w))
    fl = 2.0 * 32 * 2048 * 8192
    out["c2"] = {"sample": "32 of 4096 rows, whole W", "tflops": fl / many / 1e12, "tflops_single_thread": fl / one / 1e12}
    # config 3: one (batch, kv head) group of 4 query heads at S = 512, causal
    q3, k3, v3 = rng.standard_normal((1, 4, 512, 64)), rng.standard_normal((1, 1, 512, 64)), rng.standard_normal((1, 1, 512, 64))
    many, one = both(lambda: orc.sdpa(q3, k3, v3, is_causal=True, enable_gqa=True))
    fl = 4.0 * 4 * 512 * 512 * 64 / 2
    out["c3"] = {"sample": "one kv head (4 query heads), S = 512 of 4096, causal", "tflops": fl / many / 1e12,
                 "tflops_single_thread": fl / one / 1e12}
    # config 4: one decode step of the full architecture, batch 1, bf16 weights, 64 cached keys
    cfg = dict(vocab=128256, layers=16, hidden=2048, q_heads=32, kv_heads=8, head_dim=64, ffn=8192)
    bits = lambda r, c: rng.integers(0x3c00, 0x3c80, size=(r, c), dtype=np.uint16)
    H, F, V = 2048, 8192, 128256
    w = dict(embed=bits(V, H), final_norm=bits(1, H)[0], attn_norm=[bits(1, H)[0]] * 16, mlp_norm=[bits(1, H)[0]] * 16)
    for nm, (r, c) in dict(wq=(2048, H), wk=(512, H), wv=(512, H), wo=(H, 2048), wgate=(F, H), wup=(F, H), wdown=(H, F)).items():
        w[nm] = [bits(r, c)] * 16
    o = orc.Llama(dict(cfg, ctx=64, batch=1, w4=0, group=64, round_acts=1, llama3_rope=1), w)
    tok = np.zeros(1, dtype=np.int32)
    many, one = both(lambda: o.step(tok, 1))
    out["c4"] = {"sample": "one step, batch 1, bf16 weights, 64-key cache", "tok_per_s": 1.0 / many, "tok_per_s_single_thread": 1.0 / one}
    return out


# ───────────────────────── single-GPU suite (other configurations) ─────────────────────────
def time_events(fn, steps, warmup, torch):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2] * 1e-3, ts[0] * 1e-3


def suite(dev, torch, hbm_peak, tf_peak, quick, only=None, c2_shape=(4096, 2048, 8192), c3_shape=(8, 4096), fused=True, form="auto",
          c4_layers=0):
    import numpy as np
    from sanic_b200 import llama
    out = {}
    want = lambda name: only is None or any(o in name for o in only)
    td = dev.torch_device
    g = torch.Generator(device=td)
    g.manual_seed(7)
    # config 1: f32 naive attention Q[256x64] K,V[1024x64] (launch-latency bound parity case)
    if want("c1"):
        q = torch.randn(1, 1, 256, 64, generator=g, device=td)
        k = torch.randn(1, 1, 1024, 64, generator=g, device=td)
        v = torch.randn(1, 1, 1024, 64, generator=g, device=td)
        # a ~10 us kernel: time the C-ABI call itself, 20 launches between two events, so that the interval holds the
        # kernel and not the Python wrapper's tensor allocation and argument marshalling
        import ctypes as C
        o1 = torch.empty(1, 1, 256, 64, device=td)
        p1 = dev._attn_params(q, k, v, o1, False, 0, 0.125, None, 1)
        def c1_batch():
            for _ in range(20):
                dev.lib.sanic_attn_fwd_f32(dev.h, C.byref(p1), dev.stream())
        med, best = time_events(c1_batch, 10, 3, torch)
        med_call, _ = time_events(lambda: dev.attn_fwd_f32(q, k, v, scale=0.125), 20, 3, torch)
        out["c1_attn_f32_us"] = {"median": med / 20 * 1e6, "min": best / 20 * 1e6, "through_python_wrapper": med_call * 1e6}
        # the same config through the generic emitter (the fallback for carriers no hand-written kernel matches): one
        # generated kernel that reads only Q, K, V, as a scalar fold and as a cooperative fold with the value-feature axis
        # over the lanes and the key axis over 8 warps
        from sanic_b200 import emitter as em
        grid, n_keys, operands, carrier = em.attention(1, 1, 1, 256, 1024, 64, 64, 0.125)
        og = torch.empty(256 * 64, device=td)
        for label, kw in (("generated_scalar_fold", dict(lanes=1)), ("generated_cooperative_fold", dict(lanes=32, warps=8, lane_axis=True))):
            kern = em.GenericKernel(dev, em.Description(grid, operands, carrier=carrier, stream=n_keys, **kw))
            bufs = (C.c_void_p * 3)(q.data_ptr(), k.data_ptr(), v.data_ptr())
            def gen_batch():
                for _ in range(20):
                    dev.lib.sanic_generic_launch(dev.h, kern.h, bufs, 3, C.c_void_p(og.data_ptr()), dev.stream())
            med_g, _ = time_events(gen_batch, 5, 2, torch)
            out["c1_attn_f32_us"][label] = med_g / 20 * 1e6
            out["c1_attn_f32_us"][label + "_max_abs_diff"] = float((og.view(256, 64) - o1.view(256, 64)).abs().max())
            kern.close()
    # config 2: RMSNorm-fused GEMM, x[4096x2048] g[2048] W[2048x8192] bf16, f32 accumulation, bf16 output
    M, K, N = c2_shape
    x = torch.randn(M, K, generator=g, device=td).to(torch.bfloat16)
    gam = (1.0 + 0.1 * torch.randn(K, generator=g, device=td)).to(torch.bfloat16)
    for name, nk in (("w_nk", True), ("w_kn", False)):
        if not want("c2"):
            continue
        w = (0.02 * torch.randn((N, K) if nk else (K, N), generator=g, device=td)).to(torch.bfloat16)
        med, best = time_events(lambda: dev.gemm_rmsnorm(x, gam, w, w_is_nk=nk), 20, 3, torch)
        dev.sync()
        fl = 2.0 * M * N * K
        out[f"c2_gemm_rmsnorm_{name}"] = {"us_median": med * 1e6, "us_min": best * 1e6, "tflops": fl / med / 1e12,
                                          "frac_of_bf16_peak": fl / med / 1e12 / tf_peak}
        if nk:
            # weights bound once: g folded into W by a separate pass (timed on its own), the contraction then takes x as loaded
            ws = dev.gemm_prescale_weights(gam, w, w_is_nk=True)
            med_p, _ = time_events(lambda: dev.gemm_prescale_weights(gam, w, w_is_nk=True), 10, 3, torch)
            med_s, best_s = time_events(lambda: dev.gemm_rmsnorm(x, None, ws, w_is_nk=True), 20, 3, torch)
            dev.sync()
            out["c2_gemm_rmsnorm_prescaled_weights"] = {"us_median": med_s * 1e6, "us_min": best_s * 1e6, "prescale_us": med_p * 1e6,
                                                       "tflops": fl / med_s / 1e12, "tflops_with_prescale_every_call": fl / (med_s + med_p) / 1e12,
                                                       "frac_of_bf16_peak": fl / med_s / 1e12 / tf_peak}
            del ws
        del w
    del x
    if only is not None and want("c2_profile"):
        # clock counters of the pair tile with A through registers (one launch, SM pair 0): what its roles wait for
        M, K, N = c2_shape
        x = torch.randn(M, K, generator=g, device=td).to(torch.bfloat16)
        gam = (1.0 + 0.1 * torch.randn(K, generator=g, device=td)).to(torch.bfloat16)
        w = (0.02 * torch.randn(N, K, generator=g, device=td)).to(torch.bfloat16)
        for _ in range(3):
            prof, _y = dev.gemm_rmsnorm_pair_profile(x, gam, w, w_is_nk=True)
        out["c2_pair_registers_profile"] = {k: ({a: round(b, 1) for a, b in v.items()} if isinstance(v, dict) else round(v, 1)) for k, v in prof.items()}
        del x, w
    # config 3: causal flash attention with RoPE, B8 Hq32 Hkv8 D64 S4096 bf16 (+ 1024-token window)
    Bq, Hq3, Hk3, S3 = c3_shape[0], 32, 8, c3_shape[1]
    c3_scale = (Bq * S3 * S3) / (8.0 * 4096 * 4096)
    q3 = torch.randn(Bq, Hq3, S3, 64, generator=g, device=td).to(torch.bfloat16)
    k3 = torch.randn(Bq, Hk3, S3, 64, generator=g, device=td).to(torch.bfloat16)
    v3 = torch.randn(Bq, Hk3, S3, 64, generator=g, device=td).to(torch.bfloat16)
    table = dev.rope_table([math.exp(i * (-math.log(500000.0) / 32)) for i in range(32)], S3)
    qr, kr = torch.empty_like(q3), torch.empty_like(k3)
    med_r, _ = time_events(lambda: (dev.rope_bf16(q3, table, out=qr), dev.rope_bf16(k3, table, out=kr)), 10, 3, torch)
    if only is not None and "c3_profile" in only:
        # clock counters of the flash forward's softmax warps and MMA thread (one launch, CTA 0)
        for _ in range(3):
            prof, _o = dev.attn_fwd_bf16_profile(qr, kr, v3, causal=True)
        out["c3_flash_profile"] = {k: {a: ({x: round(y, 1) for x, y in b.items()} if isinstance(b, dict) else b) for a, b in v.items()}
                                   for k, v in prof.items()}
    for name, win, fl in (("causal", 0, 5.498e11 * c3_scale), ("causal_window1024", 1024, 2.405e11 * c3_scale)):
        if not want("c3"):
            continue
        med, best = time_events(lambda: dev.attn_fwd_bf16(qr, kr, v3, causal=True, window=win), 10, 3, torch)
        dev.sync()
        # the configuration includes RoPE on Q and K: the headline fraction divides by attention + RoPE time
        out[f"c3_flash_{name}"] = {"attn_us_median": med * 1e6, "attn_us_min": best * 1e6, "rope_us": med_r * 1e6,
                                   "tflops_attn_only": fl / med / 1e12, "tflops_with_rope": fl / (med + med_r) / 1e12,
                                   "frac_of_bf16_peak": fl / (med + med_r) / 1e12 / tf_peak,
                                   "frac_of_bf16_peak_attn_only": fl / med / 1e12 / tf_peak}
    del q3, k3, v3, qr, kr
    torch.cuda.empty_cache()
    if want("probe"):
      try:
        # measured device facts behind the bounds quoted for config 3 (exponentials per clock per SM, and what the softmax
        # warps' other instructions add) and for the HBM-bound folds (a read-only sweep of 4 GiB)
        import ctypes as C
        pr = {}
        for warps in (4, 8):       # 16 warps of this probe (128 live values per lane) do not fit one SM's register file
            for mode, label in enumerate(("ex2", "ex2+fma", "ex2+fma+sum", "ex2+fma+sum+pack", "quarter_on_fma_pipe", "half_on_fma_pipe",
                                          "f16x2_ex2+fma", "f16x2_ex2+fma+sum+bf16_pack", "f16x2_ex2+fma+sum",
                                          "ex2+fma+sum+pack+max3", "ex2+fma+sum+pack+two_max")):
                rate, clk = C.c_double(0.0), C.c_double(0.0)
                dev._check(dev.lib.sanic_probe_sfu(dev.h, warps, mode, 200, dev.stream(), C.byref(rate), C.byref(clk)), "probe_sfu")
                pr[f"warps{warps}_{label}"] = {"exp_per_clk_per_sm": round(rate.value, 2), "clk_per_128_per_lane": clk.value}
        buf = torch.empty(1 << 30, dtype=torch.int32, device=td)
        buf.zero_()
        gbs = C.c_double(0.0)
        dev._check(dev.lib.sanic_probe_stream(dev.h, C.c_void_p(buf.data_ptr()), buf.numel() * 4, 5, dev.stream(), C.byref(gbs)), "probe_stream")
        pr["read_only_sweep_gbs"] = round(gbs.value, 1)
        del buf
        torch.cuda.empty_cache()
        out["probe"] = pr
      except Exception as e:      # a probe must not take the rest of the suite with it
        out["probe"] = {"error": repr(e)}
    # the decode step's contractions one by one, bf16 and int4-g64 weights at batch 1 and 16: back to back in a CUDA graph,
    # weight sets in rotation (more than L2 holds), so each figure is the stand-alone kernel's own streaming rate without the
    # step's launch-to-launch gaps. Not part of the default suite: name it with --only c4_contractions, or one case of it as
    # --only c4_contractions_int4_g64_b1_lm_head (weights, batch, contraction). SANIC_GEMV_RING=0 times the register-staged
    # kernel at batch 16.
    pick = [o for o in (only or []) if o.startswith("c4_contractions")]
    if pick:
        from sanic_b200 import abi
        res = {}
        for w4 in (False, True):
            for B in (1, 16):
                sub = {}
                for name, rows, K, dual, mb in (("qkv_3072x2048", 3072, 2048, False, 12.6), ("o_2048x2048", 2048, 2048, False, 8.4),
                                                ("gate_up_2x8192x2048", 8192, 2048, True, 67.1), ("down_2048x8192", 2048, 8192, False, 33.6),
                                                ("lm_head_128256x2048", 128256, 2048, False, 525.3)):
                    if not any(o in "c4_contractions_" + ("int4_g64" if w4 else "bf16") + f"_b{B}_" + name for o in pick):
                        continue
                    per_set = mb * (0.28125 if w4 else 1.0)                  # int4 g64: 0.5 + 2/64 bytes per weight against 2
                    nset = max(2, min(16, int(300.0 / per_set) + 1))         # at least 300 MB in rotation
                    n_mat = 2 if dual else 1
                    if w4:
                        sets = [([torch.randint(0, 256, (rows, K // 2), device=td, generator=g, dtype=torch.uint8) for _ in range(n_mat)],
                                 [(0.002 + 0.001 * torch.rand(rows, K // 64, device=td, generator=g)).to(torch.bfloat16) for _ in range(n_mat)])
                                for _ in range(nset)]
                    else:
                        sets = [([(0.02 * torch.randn(rows, K, device=td, generator=g)).to(torch.bfloat16) for _ in range(n_mat)], None)
                                for _ in range(nset)]
                    xb = torch.randn(B, K, device=td, generator=g).to(torch.bfloat16)
                    kw = dict(epilogue=abi.EPI_SILU_MUL) if dual else {}
                    for ws, sc in sets:
                        dev.gemv(xb, ws, scales=sc, **kw)
                    torch.cuda.synchronize()
                    graph, st = torch.cuda.CUDAGraph(), torch.cuda.Stream(device=td)
                    with torch.cuda.stream(st):
                        with torch.cuda.graph(graph, stream=st):
                            for _ in range(4):
                                for ws, sc in sets:
                                    dev.gemv(xb, ws, scales=sc, **kw)
                        graph.replay()
                        torch.cuda.synchronize()
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(st); graph.replay(); b.record(st)
                        torch.cuda.synchronize()
                    us = a.elapsed_time(b) / (4 * nset) * 1e3
                    nbytes = n_mat * rows * (K // 2 + K // 64 * 2 if w4 else K * 2)
                    sub[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac_of_hbm_peak": round(nbytes / us / 1e3 / hbm_peak, 3)}
                    del sets, graph
                    torch.cuda.empty_cache()
                if sub:
                    res[("int4_g64" if w4 else "bf16") + f"_b{B}"] = sub
        out["c4_contractions"] = res
    # config 4: Llama-3.2-1B-architecture decode step, ctx 1024 (+32 steps), CUDA-graph replays
    cfg = dict(llama.LLAMA_3_2_1B)
    if c4_layers:       # a shallower stack of the same layers (small cases for profiling)
        cfg["layers"] = c4_layers
    for name, batch, w4 in (("bf16_b1", 1, False), ("bf16_b16", 16, False), ("int4_b1", 1, True), ("int4_b16", 16, True)):
        if not want("c4_" + name):
            continue
        w = llama.random_weights(cfg, 11, td, w4=w4)
        # the captured launch list measures faster than the step as one cooperative kernel in all four cases (batch 1: 0.810
        # against 0.858 ms with bf16 weights, 0.657 against 0.776 with int4; batch 16: 1.02 against 1.91 ms)
        persistent = fused and form == "persistent"
        # SANIC_LLAMA_DEFERRED_NORM=0/1 forces the deferred normaliser off / on (A/B timing); default: the machine's choice
        force = os.environ.get("SANIC_LLAMA_DEFERRED_NORM")
        m = llama.LlamaMachine(dev, cfg, w, ctx=1088, batch=batch, w4=w4, fused=fused, persistent=persistent,
                               deferred_norm=None if force is None else force != "0")
        deferred = m.deferred_norm
        rng = np.random.default_rng(3)
        # prefill 1024 positions from random token ids by decoding on the device
        for p in range(1024 if not quick else 64):
            if p % 64 == 0:
                m.set_state(rng.integers(0, cfg["vocab"], size=batch).astype(np.int32), p)
            m.step()
        m.sync()
        m.set_state(rng.integers(0, cfg["vocab"], size=batch).astype(np.int32), 1024)
        for _ in range(3):
            m.step()
        m.sync()
        secs = [m.step(timed=True) for _ in range(32)]
        sec = sorted(secs)[len(secs) // 2]
        kv_bytes = batch * cfg["layers"] * 2 * cfg["kv_heads"] * 1040 * cfg["head_dim"] * 2
        wb = m.weight_bytes()
        if want("c4_profile") and persistent:
            # per phase: [activations staged, last contraction done, sums + epilogue done, barrier released] (us, block 0)
            prof = m.step_phase_profile()
            m.sync()
            out[f"c4_phase_profile_{name}"] = [[round(t * 1e6, 2) for t in ph] for ph in prof]
        out[f"c4_llama_decode_{name}"] = {
            "tok_per_s": batch / sec, "ms_per_step": sec * 1e3, "launches_per_step": m.kernel_count,
            "form": ("one cooperative kernel" if m.kernel_count == 1 else "one cooperative kernel, then the vocabulary contraction and the token choice as launches")
                    if persistent else "captured launch list", "deferred_norm": bool(deferred),
            "algorithmic_bytes": wb + kv_bytes, "achieved_gbs": (wb + kv_bytes) / sec / 1e9,
            "frac_of_hbm_peak": (wb + kv_bytes) / sec / 1e9 / hbm_peak}
        del m, w
        torch.cuda.empty_cache()
    return out


# ───────────────────────── the product arm ─────────────────────────
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import sanic_b200
    from sanic_b200.splitkv import SplitKVDecoder, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = sanic_b200.CudaDevice(local)
    td = dev.torch_device
    hbm_peak, tf_peak, peak_kind = measured_peaks()

    L = args.kv_len
    lo, hi = shard_range(L, rank, world)
    n_local = hi - lo
    g = torch.Generator(device=td)
    g.manual_seed(1000 + rank)
    k = torch.empty((B, HKV, n_local, D), dtype=torch.bfloat16, device=td)
    v = torch.empty_like(k)
    for t in (k, v):                       # chunked fill keeps the f32 temporaries small
        for b in range(B):
            for h in range(HKV):
                t[b, h].copy_(torch.randn(n_local, D, generator=g, device=td, dtype=torch.float32))
    total = args.steps + args.warmup
    gq = torch.Generator(device="cpu")
    gq.manual_seed(77)                     # the same queries on every rank
    q_host = torch.randn(total, B, HQ, D, generator=gq).to(torch.bfloat16).pin_memory()
    q_dev = q_host.to(td)
    out_host = torch.empty((B, HQ, D), dtype=torch.bfloat16).pin_memory()
    dec = SplitKVDecoder(dev, k, v, exchange="fused" if (world == 1 and args.exchange in ("auto", "fused")) else "nccl")
    # N > 1: the exchange either as an NCCL all-gather followed by the merge kernel, or as one kernel over peer memory
    # (accumulators stored into every peer's buffer over NVLink, flags, merge). The peer form is used when it can be
    # set up and gives, bit for bit, the NCCL form's output on a first step.
    exchange, exchange_note = ("nccl" if world > 1 else "none"), ""
    if world > 1 and args.exchange != "nccl":
        try:
            form = "peer" if args.exchange == "peer" else "fused"
            dec_peer = SplitKVDecoder(dev, k, v, n_splits=dec.n_splits if form == "peer" else None, init_nccl=False, exchange=form)
            o_ref = dec.step(q_dev[0]).clone()
            o_peer = dec_peer.step(q_dev[0]).clone()
            torch.cuda.synchronize()
            # the peer form merges exactly what the NCCL form merges (bit-equal); the fused form chunks the key axis
            # differently (stream-K), so it is held to one bf16 rounding of the NCCL form's output
            if form == "peer":
                agree = torch.equal(o_ref, o_peer)
            else:
                agree = bool(((o_ref.float() - o_peer.float()).abs() / (1.0 + o_ref.float().abs())).max().item() <= 2.0 ** -7)
            same = torch.tensor([1 if agree else 0], dtype=torch.int32, device=td)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            if int(same.item()) == 1:
                dec_nccl, dec, exchange = dec, dec_peer, form
            else:
                exchange_note = "peer exchange disagreed with the NCCL form; NCCL used"
        except RuntimeError as e:
            exchange_note = f"peer exchange unavailable ({e}); NCCL used"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, min_seconds):
        """Regions of EXACTLY args.steps steps, each bracketed by barrier + synchronize on both sides and timed with CUDA
        events (max over ranks). One region of 20 steps is 50 ms and ends before the clocks settle under load, so
        regions repeat until `min_seconds` of device time have been measured; the figure reported is the mean over all
        regions (rank 0 decides how many, so every rank runs the same count)."""
        for i in range(args.warmup):
            step_fn(i)
        total, regions = 0.0, 0
        while True:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step_fn(args.warmup + i)
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=td)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            total += float(ms.item()) * 1e-3
            regions += 1
            more = torch.tensor([1 if (total < min_seconds and regions < args.max_regions) else 0], dtype=torch.int32, device=td)
            if world > 1:
                dist.broadcast(more, src=0)
            if int(more.item()) == 0:
                break
        return total / regions, regions

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # device-resident inputs
    sec, regions = timed(lambda i: dec.step(q_dev[i]), args.min_seconds)

    # end to end through the public call: q from pinned host memory, result read back to the host
    def e2e_step(i):
        qd = q_host[i].to(td, non_blocking=True)
        o = dec.step(qd)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    sec_e2e, regions_e2e = timed(e2e_step, args.min_seconds / 2)
    clocks = sampler.stop() if rank == 0 else None

    # dominant kernel alone (the local fold), live CUDA events on the launching stream
    import ctypes as C
    car = torch.empty((B * HQ, D + 2), dtype=torch.float32, device=td)
    p, _keep = dev.decode_params(q_dev[0], k, v, n_local, n_splits=dec.n_splits, carrier_out=car)
    fold_fn = dev.lib.sanic_attn_decode_streamk if dec.exchange == "fused" else dev.lib.sanic_attn_decode_splitkv
    def fold_only():
        dev._check(fold_fn(dev.h, C.byref(p), dev.stream()), "decode")
    evs = []
    for i in range(3 + args.steps):
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fold_only(); b_.record()
        if i >= 3:
            evs.append((a, b_))
    torch.cuda.synchronize()
    kt = torch.tensor([sum(a.elapsed_time(b_) for a, b_ in evs) / len(evs) * 1e-3], device=td)
    if world > 1:
        dist.all_reduce(kt, op=dist.ReduceOp.MAX)
    kern_sec = float(kt.item())

    bytes_total = 2 * B * HKV * L * D * 2
    bytes_local = 2 * B * HKV * n_local * D * 2
    line = None
    if rank == 0:
        achieved = bytes_local / kern_sec / 1e9
        line = {
            "metric": METRIC, "value": bytes_total * args.steps / sec / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"split-KV decode attention B{B} Hq{HQ} Hkv{HKV} D{D} bf16, {L} keys/sequence "
                                   f"sharded over {world} GPU(s) on the sequence axis",
                       "kv_bytes_total": bytes_total, "n_splits_per_gpu": dec.n_splits,
                       "l2": "inputs larger than L2 (>= 2 GB per GPU per step), no flush needed",
                       "timed_regions": regions, "timed_regions_e2e": regions_e2e,
                       "timing": f"{regions} regions of {args.steps} steps each (barrier + synchronize around every region, CUDA "
                                 f"events, max over ranks), mean over regions: at least {args.min_seconds} s of device time so that "
                                 "the clocks under sustained load are the ones sampled",
                       "headline": ("e2e: with more than one GPU `value` times back-to-back steps, where a rank's exchange hides "
                                    "under its next fold; `e2e` synchronises every step, as a token-feedback loop does")
                                   if world > 1 else "e2e (value and roofline explain it)",
                       "exchange": {"none": "none (1 GPU)", "nccl": "NCCL all-gather of (m,l,o) carriers + derived combine",
                                    "peer": "a second kernel: peer stores of (m,l,o) carriers over NVLink + flags + derived combine (bit-identical to the NCCL form)",
                                    "fused": "none beyond the fold's own launch: its last arrivers store (m,l,o) carriers into every peer over NVLink, flag, wait and merge per (batch, kv head) group"}[exchange],
                       **({"exchange_note": exchange_note} if exchange_note else {})},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": TRAFFIC_RATIO_DECODE * bytes_local if TRAFFIC_RATIO_DECODE else None,
                         "kernel": "attn_decode_streamk_kernel<128,false>" if dec.exchange == "fused" else "attn_decode_kernel<128,false>", "peak_kind": f"of {peak_kind}",
                         "kernel_ms": kern_sec * 1e3, "algorithmic_bytes_per_launch": bytes_local},
            "e2e": {"value": bytes_total * args.steps / sec_e2e / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": B * HQ * D * 2, "d2h_bytes_per_step": B * HQ * D * 2,
                    "ms_per_step": sec_e2e / args.steps * 1e3},
            "gpu_launches": args.steps * regions * (1 if (world == 1 or exchange == "fused") else 2),      # every region of the device-timed figure
            "clocks": clocks,
        }
        if not args.no_cpu and world == 1:
            gbs, csec, threads = cpu_sample(args.cpu_sample_keys, 1)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"{args.cpu_sample_keys} of {L} keys per sequence, all {B}x{HQ} heads, "
                                              f"dense f64 oracle, {csec:.2f} s"}
            # the reference's interpreter is single-threaded: the same path on one thread, on a quarter of the sample
            from oracle import oracle as orc
            orc.set_num_threads(1)
            gbs1, csec1, _ = cpu_sample(max(256, args.cpu_sample_keys // 4), 1)
            orc.set_num_threads(threads)
            line["cpu_baseline"]["single_thread"] = {"value": gbs1, "unit": "GB/s", "cores": 1,
                                                     "sample": f"{max(256, args.cpu_sample_keys // 4)} keys per sequence, {csec1:.2f} s"}
    del dec, k, v
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_suite and not args.no_cpu:
        try:
            line["cpu_baseline"]["suite"] = cpu_suite()
        except Exception as e:
            line["cpu_baseline"]["suite"] = {"error": repr(e)}
    if rank == 0 and world == 1 and not args.no_suite:
        try:
            line["suite"] = suite(dev, torch, hbm_peak, tf_peak, args.quick, args.only.split(",") if args.only else None,
                                  tuple(int(t) for t in args.c2_shape.split(",")), tuple(int(t) for t in args.c3_shape.split(",")), not args.llama_unfused, args.llama_form, args.c4_layers)
        except Exception as e:  # the headline line must still print
            line["suite"] = {"error": repr(e)}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# dram bytes (read + write) / algorithmic bytes of the decode fold, from one ncu capture of a 65,536-key case (1.0740 GB read
# + 7.9 MB written for 1.0737 GB of K and V); the traffic grows in proportion to the keys streamed
TRAFFIC_RATIO_DECODE = 1.0076


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--min-seconds", type=float, default=2.0, help="repeat the timed region of `steps` steps until this much device time is measured")
    ap.add_argument("--max-regions", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kv-len", type=int, default=L_FULL)
    ap.add_argument("--cpu-sample-keys", type=int, default=4096)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-suite", action="store_true")
    ap.add_argument("--quick", action="store_true", help="shorter prefill in the suite")
    ap.add_argument("--only", default="", help="comma-separated substrings of suite entries to run (c1,c2,c3,c4_bf16_b1,...); entries outside the default suite "
                         "run only when named: c2_profile, c3_profile, c4_contractions[_<weights>_b<batch>[_<name>]]")
    ap.add_argument("--c2-shape", default="4096,2048,8192", help="M,K,N of the suite's GEMM (small cases for profiling)")
    ap.add_argument("--llama-unfused", action="store_true", help="one stage per graph cone in the decode step")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "peer", "fused"], help="how N > 1 ranks exchange their accumulators")
    ap.add_argument("--llama-form", default="auto", choices=["auto", "list", "persistent"],
                    help="decode step as the captured launch list, as one cooperative kernel, or whichever measured faster for the batch")
    ap.add_argument("--c4-layers", type=int, default=0, help="layers of the suite's decode-step model (0: the architecture's 16)")
    ap.add_argument("--c3-shape", default="8,4096", help="batch,sequence of the suite's prefill attention")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
