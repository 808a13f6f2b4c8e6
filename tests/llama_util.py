"""Test plumbing for the decode-step parity tests: host copies of the device weights in the layout the CPU oracle
takes, and the lock-step comparison of a device machine with the stateful oracle."""
import numpy as np
import torch

from oracle import oracle as orc


def weights_to_oracle(w: dict, w4: bool):
    """Host copies in the layout oracle.Llama takes (bf16 bits as uint16, packed int4 as uint8)."""
    def bits(t):
        return t.view(torch.int16).cpu().numpy().view("uint16")

    head_w4 = w["embed"].dtype == torch.uint8
    out = dict(embed=w["embed"].cpu().numpy() if head_w4 else bits(w["embed"]), final_norm=bits(w["final_norm"]),
               attn_norm=[bits(t) for t in w["attn_norm"]], mlp_norm=[bits(t) for t in w["mlp_norm"]])
    if head_w4:
        out["sembed"] = bits(w["sembed"])
    for name in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown"):
        out[name] = [t.cpu().numpy() if w4 else bits(t) for t in w[name]]
        if w4:
            out["s" + name[1:]] = [bits(t) for t in w["s" + name[1:]]]
    return out


def make_oracle(cfg, w, ctx, batch, w4, norm_store=0):
    ocfg = dict(cfg, ctx=ctx, batch=batch, w4=int(w4), group=64, round_acts=1, llama3_rope=1,
                w4_head=int(w["embed"].dtype == torch.uint8), norm_store=norm_store)
    return orc.Llama(ocfg, weights_to_oracle(w, w4))


def prefill_on_device(machines, o, cfg, prefill, rng):
    """Fill the caches by decoding random token ids on the device (first machine), then hand the bf16 cache
    contents to the oracle and to the other machines so every side starts the compared steps from identical state."""
    m0 = machines[0]
    toks = rng.integers(0, cfg["vocab"], size=(prefill, m0.batch)).astype(np.int32)
    for p in range(prefill):
        m0.set_state(toks[p], p)
        m0.step()
    m0.sync()
    for l in range(cfg["layers"]):
        o.kcache[l] = m0.kcache[l].float().cpu().numpy().astype(np.float64)
        o.vcache[l] = m0.vcache[l].float().cpu().numpy().astype(np.float64)
    for m in machines[1:]:
        m.load_caches(m0.kcache, m0.vcache)


def lockstep(machines, o, cfg, prefill, steps, rng, label=""):
    """Greedy steps of every machine against the oracle. Returns (ties, worst_gap, max_logit_err) per machine.

    Logits must agree to the bf16 bound at every step. A token that differs from the oracle's is an error unless the
    oracle's own top-2 gap on that row is inside the bf16 bound (both indices are then maxima to within the storage
    precision: a tie); ties are counted and reported, and both sides continue from the oracle's token."""
    batch = machines[0].batch
    cur = rng.integers(0, cfg["vocab"], size=batch).astype(np.int32)
    for m in machines:
        m.set_state(cur, prefill)
    ocur = cur.copy()
    stats = [dict(ties=0, worst_gap=float("inf"), err=0.0, rms=0.0, min_gap=float("inf")) for _ in machines]
    # The bf16 bound of one kernel is 2e-2. The logits of the whole stack are held to it as a vector (relative rms).
    # Per element, the two sides' bf16 roundings of the activations decorrelate with depth (an f32-vs-f64 difference
    # of 1e-7 flips a rounding here and there, each flip moves later roundings): the difference then looks like the
    # rounding noise of the model itself, independent per layer, so the largest of the vocabulary's normalised
    # differences is bounded by the single-kernel bound times the square root of the depth (a 2-layer model: 2.8e-2,
    # 16 layers: 8e-2; measured on the 16-layer architecture: 4.3e-2 to 5.8e-2 with bf16 weights, 6e-4 with int4).
    # The largest of N such differences grows like sqrt(2 ln N): the figures above are for one row of the vocabulary
    # (N = 128256); a batch of rows is held to the same noise level, i.e. to the bound scaled by sqrt(ln N / ln 128256)
    # (batch 16: 1.11; measured there: up to 8.2e-2 over 32 steps).
    n_el = batch * cfg["vocab"]
    tol_logits = 2e-2 * max(1.0, cfg["layers"] ** 0.5) * max(1.0, (np.log(n_el) / np.log(128256.0)) ** 0.5)
    for s in range(steps):
        for m in machines:
            m.step()
        ocur = o.step(ocur, prefill + s)
        ol = o.logits()
        top = np.sort(ol, axis=1)
        gaps_all = top[:, -1] - top[:, -2]
        for m, st in zip(machines, stats):
            got = m.read_tokens()
            lg = m.logits.cpu().numpy().astype(np.float64)
            err = np.max(np.abs(lg - ol) / (1.0 + np.abs(ol)))
            assert err <= tol_logits, f"{label} step {s}: logits differ by {err}"
            rms = np.linalg.norm(lg - ol) / np.linalg.norm(ol)
            assert rms <= 2e-2, f"{label} step {s}: logits differ by {rms} in relative rms"
            st["err"] = max(st["err"], float(err))
            st["rms"] = max(st["rms"], float(rms))
            st["min_gap"] = min(st["min_gap"], float(gaps_all.min()))
            bad = np.nonzero(got != ocur)[0]
            if bad.size:
                gaps = gaps_all[bad]
                tol = 2e-2 * (1.0 + np.abs(top[bad, -1]))
                assert np.all(gaps <= tol), f"{label} step {s}: tokens {got[bad]} vs oracle {ocur[bad]}, oracle top-2 gaps {gaps}"
                assert np.all(np.abs(ol[bad, got[bad]] - top[bad, -1]) <= tol)
                st["ties"] += int(bad.size)
                st["worst_gap"] = min(st["worst_gap"], float(gaps.min()))
                if s + 1 < steps:
                    m.set_state(ocur, prefill + s + 1)      # continue both sides from the same token
    return stats


def run_pair(dev, cfg, ctx, batch, w4, steps, prefill, seed=5, fused=True, persistent=False, deferred_norm=None):
    from sanic_b200 import llama
    w = llama.random_weights(cfg, seed, dev.torch_device, w4=w4)
    m = llama.LlamaMachine(dev, cfg, w, ctx=ctx, batch=batch, w4=w4, fused=fused, persistent=persistent, deferred_norm=deferred_norm)
    # the oracle rounds where the machine does: stored(bf16) on x * gamma at the deferred norms
    o = make_oracle(cfg, w, ctx, batch, w4, norm_store=2 if m.deferred_norm else 0)
    rng = np.random.default_rng(seed)
    prefill_on_device([m], o, cfg, prefill, rng)
    st = lockstep([m], o, cfg, prefill, steps, rng)[0]
    assert st["ties"] <= max(1, steps * batch // 16), f"{st['ties']} near-tie steps out of {steps * batch}"
    return m
