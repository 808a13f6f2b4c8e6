"""Decode-step parity: the captured launch list against the stateful CPU oracle.

Greedy tokens must be identical step for step; logits agree to the bf16 bound. Both sides round
at the same declared storage points (weights, caches, projection inputs and q in bf16; residual
stream f32); the remaining differences are f32-vs-f64 accumulation and the bf16 rounding of the
attention probabilities that feed the tensor-core P.V product. When a token differs the
test prints the oracle's top-2 logit gap: a gap below the bf16 bound is a tie, not an error.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from llama_util import run_pair

pytestmark = pytest.mark.gpu

SMALL = dict(vocab=1024, layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512)


@pytest.fixture(scope="module")
def dev():
    from sanic_b200 import CudaDevice
    return CudaDevice(0)


@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("w4", [False, True])
def test_small_model_32_greedy_steps(dev, batch, w4):
    run_pair(dev, SMALL, ctx=128, batch=batch, w4=w4, steps=32, prefill=40)


@pytest.mark.parametrize("w4", [False, True])
def test_small_model_one_stage_per_cone(dev, w4):
    # the unfused launch list (norm, projections, RoPE + cache write as separate stages: 8 per layer)
    m = run_pair(dev, SMALL, ctx=128, batch=2, w4=w4, steps=32, prefill=40, fused=False)
    assert m.n_stages == 1 + 8 * SMALL["layers"] + 4


@pytest.mark.parametrize("batch,w4", [(1, False), (3, True), (16, False)])
def test_single_kernel_step(dev, batch, w4):
    # the same stage list lowered into one cooperative kernel with grid barriers between the stages
    m = run_pair(dev, SMALL, ctx=128, batch=batch, w4=w4, steps=32, prefill=40, persistent=True)
    assert m.kernel_count == 1
    times = m.step_stage_times()
    assert len(times) == m.n_stages + 1 and all(t >= 0.0 for t in times)      # argmax is two phases
    assert m.n_stages == 1 + 5 * SMALL["layers"] + 3       # norms ride the projections at any batch in this form


def test_batch16_and_replay_equals_eager(dev):
    from sanic_b200 import llama
    m = run_pair(dev, SMALL, ctx=64, batch=16, w4=False, steps=8, prefill=10)
    # a captured replay and an eager run of the same stage list give identical tokens
    w = m.w
    a = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=16, capture=True)
    b = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=16, capture=False)
    start = np.arange(16, dtype=np.int32)
    a.set_state(start, 0); b.set_state(start, 0)
    for _ in range(12):
        a.step(); b.step()
    assert np.array_equal(a.read_tokens(), b.read_tokens())
    assert int(a.position.item()) == 12
    assert a.kernel_count == a.n_stages + 1
    # batch 16: only layer 0's attention norm stays a stage of its own (the others are deferred across the contractions)
    assert a.deferred_norm and a.n_stages == 1 + 1 + 5 * SMALL["layers"] + 3
    c = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=16, deferred_norm=False)
    assert c.n_stages == 1 + 7 * SMALL["layers"] + 4      # without it: both norms of every layer are stages


def test_machine_refuses_bad_state(dev):
    from sanic_b200 import CompileError, RunError, llama
    w = llama.random_weights(SMALL, 1, dev.torch_device)
    m = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=1)
    with pytest.raises(RunError):
        m.set_state([0], 64)
    with pytest.raises(CompileError):
        llama.LlamaMachine(dev, dict(SMALL, hidden=128), w, ctx=64, batch=1)


def test_generate_matches_manual_stepping(dev):
    # the greedy loop: prompt consumed through the decode step, then device-side feedback only
    from sanic_b200 import llama
    w = llama.random_weights(SMALL, 21, dev.torch_device)
    prompts = np.array([[5, 17, 900, 3], [1, 2, 3, 4]], dtype=np.int32)
    m = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=2)
    got = m.generate(prompts, 10)
    m2 = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=2)
    for pos in range(3):
        m2.set_state(prompts[:, pos], pos)
        m2.step()
    m2.set_state(prompts[:, 3], 3)
    want = []
    for _ in range(10):
        m2.step()
        want.append(m2.read_tokens())
    assert got.tolist() == np.array(want).T.tolist()
    with pytest.raises(llama.RunError):
        m.generate(prompts, 100)


def test_text_in_text_out(dev):
    """The loop of the reference's example around the machine (examples/llama3_2.rs:454-470, 577-681): the prompt is
    tokenized with its begin-of-text token, consumed through the decode step, and each generated id is decoded back to
    text. Random weights give no language, so what is checked is the plumbing: the oracle stepping over the same ids
    agrees with the generated ones (up to counted near-ties), both machine forms agree, and the text round-trips."""
    from sanic_b200 import llama
    from sanic_b200.tokenizer import Tokenizer
    from llama_util import make_oracle
    from test_tokenizer import SAMPLE, learn, spec
    tok = Tokenizer(spec(learn(SAMPLE, 120)))
    size = len(tok.vocab) + len(tok.added)
    cfg = dict(SMALL, vocab=-(-size // 16) * 16)
    prompt = "the cache grows by one row per step"
    ids = tok.encode(prompt, add_special_tokens=True)
    assert ids[0] == tok.added["<|begin_of_text|>"] and tok.decode(ids) == prompt
    new = 12
    w = llama.random_weights(cfg, 11, dev.torch_device)
    outs = []
    for persistent in (False, True):
        m = llama.LlamaMachine(dev, cfg, w, ctx=64, batch=1, persistent=persistent)
        outs.append(m.generate([ids], new)[0])
    assert np.array_equal(outs[0], outs[1])
    o = make_oracle(cfg, w, 64, 1, False)
    cur, differ = None, 0
    for pos, t in enumerate(ids):
        cur = o.step(np.array([t], dtype=np.int32), pos)
    for i in range(new):
        differ += int(cur[0] != outs[0][i])
        cur = o.step(np.array([outs[0][i]], dtype=np.int32), len(ids) + i)      # follow the device's ids
    assert differ <= 1
    known = [int(t) for t in outs[0] if int(t) in tok.id_to_token]
    text = tok.decode(known)
    assert isinstance(text, str) and tok.decode(tok.encode(text, False)) == text


@pytest.mark.parametrize("batch,w4,persistent", [(1, False, False), (3, True, False), (16, False, False), (16, True, False),
                                                 (1, False, True), (2, True, True), (16, False, True)])
def test_deferred_normaliser(dev, batch, w4, persistent):
    """RMSNorm split across two contractions: the residual-add epilogue writes bf16(x * gamma) and per-tile sums of x^2,
    the next contraction multiplies its outputs by 1/sqrt(mean + eps). The oracle moves its stored(bf16) point with it
    (norm_store = 2) and the tokens must agree step for step, in the launch list and in the single-kernel form."""
    m = run_pair(dev, SMALL, ctx=128, batch=batch, w4=w4, steps=32, prefill=40, persistent=persistent, deferred_norm=True)
    L = SMALL["layers"]
    first_norm = 0 if (batch <= 4 or persistent) else 1          # layer 0's attention norm: inlined, or a stage of its own
    assert m.n_stages == 1 + first_norm + 5 * L + 3
