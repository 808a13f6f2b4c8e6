"""safetensors checkpoints: the header parser and its refusals on CPU; on the GPU, a random-init model of the Llama
architecture written under the checkpoint's names, read back through per-tensor uploads from file offsets, bit for bit,
and decoding the same tokens as the model built from the tensors directly."""
import json
import os
import struct

import numpy as np
import pytest

from sanic_b200 import checkpoint as ck


def small_file(tmp_path, pad_header=True):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = (np.arange(10, dtype=np.uint16) * 257).reshape(2, 5)
    path = str(tmp_path / "t.safetensors")
    ck.write(path, {"a": ("F32", a), "b.weight": ("BF16", b)}, metadata={"format": "pt"})
    return path, a, b


def test_round_trip_and_offsets(tmp_path):
    path, a, b = small_file(tmp_path)
    entries, data_start, meta = ck.read_header(path)
    assert meta == {"format": "pt"} and data_start % 8 == 0
    assert entries["a"] == ("F32", (3, 4), 0, 48) and entries["b.weight"] == ("BF16", (2, 5), 48, 68)
    c = ck.Checkpoint(path)
    assert np.array_equal(c.host_view("a"), a) and np.array_equal(c.host_view("b.weight"), b)
    with pytest.raises(ck.CheckpointError):
        c.host_view("missing")
    c.close()


def rewrite_header(path, mutate):
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    mutate(header)
    text = json.dumps(header).encode()
    open(path, "wb").write(struct.pack("<Q", len(text)) + text + raw[8 + n:])


@pytest.mark.parametrize("what", ["dtype", "length", "overlap", "hole", "trailing", "truncated", "not json", "huge header"])
def test_malformed_files_are_refused(tmp_path, what):
    path, a, b = small_file(tmp_path)
    if what == "dtype":
        rewrite_header(path, lambda h: h["a"].update(dtype="F13"))
    elif what == "length":
        rewrite_header(path, lambda h: h["a"].update(shape=[3, 5]))
    elif what == "overlap":
        rewrite_header(path, lambda h: h["b.weight"].update(data_offsets=[40, 60]))
    elif what == "hole":
        rewrite_header(path, lambda h: (h["a"].update(shape=[11], data_offsets=[0, 44])))
    elif what == "trailing":
        open(path, "ab").write(b"\0" * 4)
    elif what == "truncated":
        raw = open(path, "rb").read()
        open(path, "wb").write(raw[:-6])
    elif what == "not json":
        raw = open(path, "rb").read()
        open(path, "wb").write(raw[:8] + b"{" * 8 + raw[16:])
    else:
        raw = open(path, "rb").read()
        open(path, "wb").write(struct.pack("<Q", 1 << 40) + raw[8:])
    with pytest.raises(ck.CheckpointError):
        ck.read_header(path)


def test_llama_names_cover_the_decode_graph():
    cfg = dict(vocab=1024, layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512)
    names = ck.llama_names(cfg)
    assert len(names) == 2 + 9 * cfg["layers"]
    assert names["model.layers.1.self_attn.k_proj.weight"] == (128, 256)       # [out, in], checkpoint-native
    assert names["model.layers.0.mlp.down_proj.weight"] == (256, 512)
    assert "lm_head.weight" not in names                                        # tied to the embedding


@pytest.mark.gpu
def test_llama_checkpoint_loads_bit_for_bit_and_decodes_the_same_tokens(tmp_path):
    import torch
    from sanic_b200 import CudaDevice, llama
    dev = CudaDevice(0)
    cfg = dict(vocab=1024, layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512)
    w = llama.random_weights(cfg, 5, dev.torch_device)
    path = str(tmp_path / "model.safetensors")
    ck.save_llama(path, cfg, w)
    entries, _, _ = ck.read_header(path)
    assert set(entries) == set(ck.llama_names(cfg))
    w2 = ck.load_llama(dev, path, cfg)
    for key, val in w.items():
        pairs = zip(val, w2[key]) if isinstance(val, list) else [(val, w2[key])]
        for x, y in pairs:
            assert x.dtype == y.dtype == torch.bfloat16 and torch.equal(x.view(torch.int16), y.view(torch.int16)), key
    toks = []
    for weights in (w, w2):
        m = llama.LlamaMachine(dev, cfg, weights, ctx=64, batch=2)
        m.set_state(np.array([3, 700], dtype=np.int32), 0)
        out = []
        for _ in range(12):
            m.step()
            out.append(m.read_tokens().tolist())
        toks.append(out)
    assert toks[0] == toks[1]
    # a storage mismatch is refused, not converted; so is a wrong shape
    c = ck.Checkpoint(path)
    with pytest.raises(ck.CheckpointError):
        c.upload(dev, "model.norm.weight", "F32")
    with pytest.raises(ck.CheckpointError):
        c.upload(dev, "model.norm.weight", "BF16", shape=(cfg["hidden"] + 1,))
    c.close()
    with pytest.raises(ck.CheckpointError):
        ck.load_llama(dev, path, dict(cfg, layers=3))
