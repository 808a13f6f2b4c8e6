"""safetensors checkpoints: header parse, validation, and device upload of each tensor from its in-file offset.

Mirrors what the reference's Llama example does with its checkpoint (examples/llama3_2.rs:346-380 of the
reference project: the file is read once, parsed in place, and every tensor binds at its offset) and the
weight naming of that example's graph (examples/llama3_2.rs:112-253: `model.embed_tokens.weight`,
`model.layers.{l}.self_attn.q_proj.weight`, ..., `model.norm.weight`, tied lm_head, matrices in the
checkpoint-native [out, in] layout). The format itself is public: 8 bytes little-endian header length, a JSON
header {name: {dtype, shape, data_offsets: [begin, end)}}, then the tensor bytes.

No file is shipped or fetched: tests write small files in this format and read them back. Uploads go through
`sanic_upload` of the C ABI, straight from the memory-mapped file.
"""
from __future__ import annotations

import ctypes as C
import json
import mmap
import os
import struct

import numpy as np

DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1, "U32": 4}


class CheckpointError(ValueError):
    """A malformed or unexpected checkpoint (the example's `Err(String)` paths)."""


def read_header(path: str):
    """Returns (entries, data_start, metadata): entries maps name -> (dtype, shape, begin, end) with offsets relative
    to data_start. Every entry is validated: known dtype, byte length = prod(shape) * width, inside the file, and the
    data section is covered exactly once (no overlap, no hole), as the format requires."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise CheckpointError(f"{path}: shorter than its 8-byte header length")
        (n,) = struct.unpack("<Q", head)
        if n < 2 or 8 + n > size:
            raise CheckpointError(f"{path}: header length {n} does not fit a file of {size} bytes")
        try:
            header = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise CheckpointError(f"{path}: header is not an object")
    data_start, data_len = 8 + n, size - 8 - n
    meta = header.pop("__metadata__", {})
    entries, spans = {}, []
    for name, e in header.items():
        try:
            dtype, shape, (begin, end) = e["dtype"], [int(d) for d in e["shape"]], e["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise CheckpointError(f"{path}: tensor {name!r} lacks dtype / shape / data_offsets") from None
        if dtype not in DTYPE_BYTES:
            raise CheckpointError(f"{path}: tensor {name!r} has unknown dtype {dtype!r}")
        want = DTYPE_BYTES[dtype] * int(np.prod(shape, dtype=np.int64)) if shape else DTYPE_BYTES[dtype]
        if not (0 <= begin <= end <= data_len) or end - begin != want:
            raise CheckpointError(f"{path}: tensor {name!r} spans [{begin}, {end}) but its shape needs {want} bytes of {data_len}")
        entries[name] = (dtype, tuple(shape), int(begin), int(end))
        spans.append((int(begin), int(end), name))
    spans.sort()
    at = 0
    for begin, end, name in spans:
        if begin != at:
            raise CheckpointError(f"{path}: data section has a hole or an overlap before {name!r} (offset {begin}, expected {at})")
        at = end
    if at != data_len:
        raise CheckpointError(f"{path}: {data_len - at} trailing bytes not described by the header")
    return entries, data_start, meta


def write(path: str, tensors: dict, metadata: dict | None = None):
    """Writes `tensors` (name -> (dtype string, numpy array of the raw storage)) in the format; bf16 travels as its
    uint16 bit patterns. The header is padded with spaces to a multiple of 8 bytes, as writers of the format do."""
    header, at, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr)
        if raw.dtype.itemsize != DTYPE_BYTES[dtype]:
            raise CheckpointError(f"{name!r}: storage width does not match {dtype}")
        header[name] = {"dtype": dtype, "shape": list(raw.shape), "data_offsets": [at, at + raw.nbytes]}
        at += raw.nbytes
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw.tobytes())


class Checkpoint:
    """An open, memory-mapped checkpoint. `upload(dev, name, dtype)` copies one tensor to the device from its offset."""

    def __init__(self, path: str):
        self.path = path
        self.entries, self.data_start, self.metadata = read_header(path)
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)     # private mapping: a host pointer for the ABI
        self._anchor = C.c_char.from_buffer(self._map)
        self._base = C.addressof(self._anchor)

    def names(self):
        return list(self.entries)

    def host_view(self, name: str) -> np.ndarray:
        dtype, shape, begin, end = self._entry(name)
        np_dtype = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "F64": np.float64, "I64": np.int64,
                    "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.uint8, "U32": np.uint32}[dtype]
        return np.frombuffer(self._map, dtype=np_dtype, count=(end - begin) // np.dtype(np_dtype).itemsize,
                             offset=self.data_start + begin).reshape(shape)

    def _entry(self, name):
        if name not in self.entries:
            raise CheckpointError(f"{self.path}: no tensor named {name!r}")
        return self.entries[name]

    def upload(self, dev, name: str, dtype: str, shape=None):
        """Allocates a device tensor of the entry's shape and copies the bytes at the entry's file offset into it.
        The storage dtype must be the declared one: a mismatch is refused, never converted (the storage-mismatch
        refusal of the reference's stateful path)."""
        import torch
        got, eshape, begin, end = self._entry(name)
        if got != dtype:
            raise CheckpointError(f"{self.path}: {name!r} is stored as {got}, the graph declares {dtype}")
        if shape is not None and tuple(shape) != eshape:
            raise CheckpointError(f"{self.path}: {name!r} has shape {eshape}, the graph declares {tuple(shape)}")
        tdt = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "U8": torch.uint8, "I32": torch.int32}[dtype]
        out = torch.empty(eshape, dtype=tdt, device=dev.torch_device)
        dev._check(dev.lib.sanic_upload(dev.h, C.c_void_p(out.data_ptr()), C.c_void_p(self._base + self.data_start + begin),
                                        C.c_size_t(end - begin), dev.stream()), f"upload {name}")
        return out

    def close(self):
        if getattr(self, "_map", None) is not None:
            self._anchor = None
            try:
                self._map.close()
            except BufferError:
                pass     # a numpy view is still alive; the mapping goes with it
            self._map = None
            self._file.close()


# ── the Llama decode graph's weight names (examples/llama3_2.rs:112-253) ──
_LAYER = {"attn_norm": "input_layernorm.weight", "mlp_norm": "post_attention_layernorm.weight",
          "wq": "self_attn.q_proj.weight", "wk": "self_attn.k_proj.weight", "wv": "self_attn.v_proj.weight",
          "wo": "self_attn.o_proj.weight", "wgate": "mlp.gate_proj.weight", "wup": "mlp.up_proj.weight",
          "wdown": "mlp.down_proj.weight"}


def llama_names(cfg: dict) -> dict:
    """Checkpoint name -> expected shape for the architecture `cfg` (matrices [out, in]; the lm_head is tied)."""
    H, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    Hq, Hkv, D = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
    shapes = {"attn_norm": (H,), "mlp_norm": (H,), "wq": (Hq * D, H), "wk": (Hkv * D, H), "wv": (Hkv * D, H), "wo": (H, Hq * D),
              "wgate": (F, H), "wup": (F, H), "wdown": (H, F)}
    out = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    for l in range(cfg["layers"]):
        for key, suffix in _LAYER.items():
            out[f"model.layers.{l}.{suffix}"] = shapes[key]
    return out


def load_llama(dev, path: str, cfg: dict) -> dict:
    """Reads a bf16 checkpoint of the architecture into the weight dictionary `LlamaMachine` takes. Every tensor the graph
    names must be present with the declared shape and bf16 storage; a separate `lm_head.weight` is accepted only if the
    file says so by carrying it (it is then ignored in favour of the tied embedding, as in the example)."""
    ck = Checkpoint(path)
    try:
        missing = [n for n in llama_names(cfg) if n not in ck.entries]
        if missing:
            raise CheckpointError(f"{path}: missing {len(missing)} tensors, first {missing[0]!r}")
        shapes = llama_names(cfg)
        w = dict(embed=ck.upload(dev, "model.embed_tokens.weight", "BF16", shapes["model.embed_tokens.weight"]),
                 final_norm=ck.upload(dev, "model.norm.weight", "BF16", shapes["model.norm.weight"]))
        for key in _LAYER:
            w[key] = []
        for l in range(cfg["layers"]):
            for key, suffix in _LAYER.items():
                name = f"model.layers.{l}.{suffix}"
                w[key].append(ck.upload(dev, name, "BF16", shapes[name]))
        dev.sync()      # the uploads read the mapping: finish them before it is closed
        return w
    finally:
        ck.close()


def save_llama(path: str, cfg: dict, w: dict):
    """Writes the bf16 weight dictionary of `llama.random_weights` under the checkpoint names (for tests and for handing a
    random-init model of the architecture to another runtime)."""
    import torch

    def bits(t):
        return t.detach().to(torch.bfloat16).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    tensors = {"model.embed_tokens.weight": ("BF16", bits(w["embed"])), "model.norm.weight": ("BF16", bits(w["final_norm"]))}
    for l in range(cfg["layers"]):
        for key, suffix in _LAYER.items():
            tensors[f"model.layers.{l}.{suffix}"] = ("BF16", bits(w[key][l]))
    write(path, tensors, metadata={"format": "pt"})
