"""Byte-level BPE text <-> token ids from a `tokenizer.json` description.

The reference's example hands its prompt to a third-party tokenizer library (`Tokenizer::from_file(tokenizer.json)`,
`.encode(prompt, true)`, and a decode of each generated id: examples/llama3_2.rs:454-470, 560-681). This module is a
restatement of the published algorithm that file describes for the Llama-3 family, so that the decode machine can be
driven from text:

  1. added (special) tokens are cut out of the text first and map straight to their ids;
  2. the rest is split by the file's pre-tokenizer regular expression;
  3. every piece is turned into its UTF-8 bytes, each byte written as one printable character of the fixed 256-entry
     byte alphabet of byte-level BPE;
  4. a piece that is a vocabulary entry as a whole is that token when the model says `ignore_merges`; otherwise adjacent
     symbols are merged, always the pair with the lowest rank in the file's merge list first (leftmost on a tie),
     until no listed pair is left;
  5. with `add_special_tokens`, the post-processor's template puts its special tokens (the begin-of-text token) around
     the ids.
Decoding inverts 3: ids -> vocabulary strings -> bytes -> UTF-8 (malformed sequences are replaced).

No vocabulary file exists in this environment; the tests build a small `tokenizer.json` of the same structure.
"""
from __future__ import annotations

import json

import regex


class TokenizerError(ValueError):
    pass


def byte_alphabet():
    """The byte <-> character table of byte-level BPE: printable Latin-1 bytes stand for themselves, the other 68 bytes
    take the code points from 256 up, in order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


_B2C = byte_alphabet()
_C2B = {c: b for b, c in _B2C.items()}


class Tokenizer:
    def __init__(self, spec: dict):
        model = spec.get("model") or {}
        if model.get("type") != "BPE":
            raise TokenizerError("load tokenizer: only a BPE model is supported")
        self.vocab = dict(model.get("vocab") or {})
        if not self.vocab:
            raise TokenizerError("load tokenizer: the model has no vocabulary")
        merges = model.get("merges") or []
        self.rank = {}
        for i, m in enumerate(merges):
            pair = tuple(m.split(" ")) if isinstance(m, str) else tuple(m)
            if len(pair) != 2:
                raise TokenizerError(f"load tokenizer: merge {i} is not a pair")
            self.rank[pair] = i
        self.ignore_merges = bool(model.get("ignore_merges", False))
        self.added = {}
        for t in spec.get("added_tokens") or []:
            self.added[t["content"]] = int(t["id"])
        self.id_to_token = {i: s for s, i in self.vocab.items()}
        for s, i in self.added.items():
            self.id_to_token[i] = s
        self.special_ids = {int(t["id"]) for t in spec.get("added_tokens") or [] if t.get("special", False)}
        self.pattern = regex.compile(self._split_pattern(spec.get("pre_tokenizer")))
        self._cut = (regex.compile("|".join(regex.escape(s) for s in sorted(self.added, key=len, reverse=True)))
                     if self.added else None)
        self.prefix, self.suffix = self._template(spec.get("post_processor"))
        self._cache = {}

    @classmethod
    def from_file(cls, path):
        try:
            with open(path, "r", encoding="utf-8") as f:
                return cls(json.load(f))
        except (OSError, json.JSONDecodeError) as e:
            raise TokenizerError(f"load tokenizer: {e}") from None

    @staticmethod
    def _split_pattern(pre):
        """The regular expression of the (first) Split step of the pre-tokenizer; a bare ByteLevel step splits on its
        own default pattern."""
        default = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
        if not pre:
            return default
        steps = pre.get("pretokenizers") if pre.get("type") == "Sequence" else [pre]
        for st in steps or []:
            if st.get("type") == "Split":
                pat = st.get("pattern") or {}
                if "Regex" in pat:
                    return pat["Regex"]
                if "String" in pat:
                    return regex.escape(pat["String"])
        return default

    def _template(self, post):
        """Ids the post-processor puts before / after a single sequence (TemplateProcessing, possibly inside a Sequence)."""
        if not post:
            return [], []
        steps = post.get("processors") if post.get("type") == "Sequence" else [post]
        for st in steps or []:
            if st.get("type") != "TemplateProcessing":
                continue
            before, after, seen = [], [], False
            for item in st.get("single") or []:
                if "Sequence" in item:
                    seen = True
                elif "SpecialToken" in item:
                    name = item["SpecialToken"]["id"]
                    ids = (st.get("special_tokens") or {}).get(name, {}).get("ids")
                    if ids is None:
                        if name not in self.added:
                            raise TokenizerError(f"load tokenizer: the template names an unknown special token {name!r}")
                        ids = [self.added[name]]
                    (after if seen else before).extend(int(i) for i in ids)
            return before, after
        return [], []

    def _bpe(self, piece: str):
        """piece: a pre-token already written in the byte alphabet -> its token ids."""
        got = self._cache.get(piece)
        if got is not None:
            return got
        if self.ignore_merges and piece in self.vocab:
            ids = [self.vocab[piece]]
        else:
            syms = list(piece)
            while len(syms) > 1:
                best, at = None, -1
                for i in range(len(syms) - 1):
                    r = self.rank.get((syms[i], syms[i + 1]))
                    if r is not None and (best is None or r < best):
                        best, at = r, i
                if best is None:
                    break
                syms[at:at + 2] = [syms[at] + syms[at + 1]]
            try:
                ids = [self.vocab[s] for s in syms]
            except KeyError as e:
                raise TokenizerError(f"tokenize prompt: symbol {e.args[0]!r} is not in the vocabulary") from None
        if len(self._cache) < 65536:
            self._cache[piece] = ids
        return ids

    def encode(self, text: str, add_special_tokens: bool = True):
        ids = []
        at = 0
        spans = list(self._cut.finditer(text)) if self._cut else []
        for m in spans + [None]:
            chunk = text[at:m.start()] if m else text[at:]
            for piece in self.pattern.findall(chunk):
                ids.extend(self._bpe("".join(_B2C[b] for b in piece.encode("utf-8"))))
            if m:
                ids.append(self.added[m.group(0)])
                at = m.end()
        return (self.prefix + ids + self.suffix) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = bytearray()
        for i in ids:
            i = int(i)
            if i not in self.id_to_token:
                raise TokenizerError(f"decode: no token has id {i}")
            s = self.id_to_token[i]
            if s in self.added:
                if not (skip_special_tokens and i in self.special_ids):
                    out.extend(s.encode("utf-8"))
                continue
            out.extend(_C2B[c] for c in s)
        return out.decode("utf-8", errors="replace")
