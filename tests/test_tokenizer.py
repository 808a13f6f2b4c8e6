"""Byte-level BPE from a tokenizer.json description (the structure the reference's example loads with its third-party
tokenizer, examples/llama3_2.rs:454-470): known answers on hand-built merge tables, round trips, special tokens and the
post-processor's begin-of-text token. The vocabulary here is synthetic: merges learnt by the test from a short sample."""
import collections
import json

import pytest

from sanic_b200.tokenizer import Tokenizer, TokenizerError, byte_alphabet

SPLIT = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
SAMPLE = ("the fold of the online softmax is a carrier of three slots ; the carrier of a contraction is one slot . "
          "a machine steps , a replay replays , and the cache grows by one row per step . 1234567 tokens , 42 heads . ") * 3


def learn(sample, n_merges):
    """A plain BPE trainer over the byte alphabet: merge the most frequent adjacent pair, n_merges times."""
    import regex
    b2c = byte_alphabet()
    words = collections.Counter("".join(b2c[b] for b in p.encode()) for p in regex.findall(SPLIT, sample))
    words = {tuple(w): c for w, c in words.items()}
    merges = []
    for _ in range(n_merges):
        pairs = collections.Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), _ = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        merges.append((a, b))
        new = {}
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and (w[i], w[i + 1]) == (a, b):
                    out.append(a + b); i += 2
                else:
                    out.append(w[i]); i += 1
            new[tuple(out)] = new.get(tuple(out), 0) + c
        words = new
    return merges


def spec(merges, ignore_merges=False, extra_vocab=()):
    b2c = byte_alphabet()
    vocab = {b2c[b]: b for b in range(256)}
    for a, b in merges:
        vocab.setdefault(a + b, len(vocab))
    for s in extra_vocab:
        vocab.setdefault(s, len(vocab))
    n = len(vocab)
    return {
        "added_tokens": [{"id": n, "content": "<|begin_of_text|>", "special": True},
                         {"id": n + 1, "content": "<|end_of_text|>", "special": True}],
        "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
            {"type": "Split", "pattern": {"Regex": SPLIT}, "behavior": "Isolated", "invert": False},
            {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False}]},
        "post_processor": {"type": "Sequence", "processors": [
            {"type": "ByteLevel"},
            {"type": "TemplateProcessing",
             "single": [{"SpecialToken": {"id": "<|begin_of_text|>", "type_id": 0}}, {"Sequence": {"id": "A", "type_id": 0}}],
             "special_tokens": {"<|begin_of_text|>": {"id": "<|begin_of_text|>", "ids": [n], "tokens": ["<|begin_of_text|>"]}}}]},
        "model": {"type": "BPE", "ignore_merges": ignore_merges, "vocab": vocab,
                  "merges": [f"{a} {b}" for a, b in merges]},
    }


def test_byte_alphabet_is_a_printable_bijection():
    t = byte_alphabet()
    assert len(t) == 256 and len(set(t.values())) == 256
    assert t[ord("a")] == "a" and t[ord("!")] == "!" and t[0xFF] == "ÿ"
    assert t[ord(" ")] == "Ġ" and t[ord("\n")] == "Ċ" and t[0] == "Ā"      # the 68 others, from 256 up in byte order
    assert all(c.isprintable() for c in t.values())


def test_merges_apply_lowest_rank_first_and_leftmost_on_ties():
    tok = Tokenizer(spec([("b", "c"), ("a", "b"), ("a", "bc")]))
    v = tok.vocab
    assert tok.encode("abc", False) == [v["abc"]]              # b+c (rank 0) first, then a+bc; a+b (rank 1) never gets its turn
    assert tok.encode("ab", False) == [v["ab"]]
    assert tok.encode("abab", False) == [v["ab"], v["ab"]]
    assert tok.encode("bcbc", False) == [v["bc"], v["bc"]]     # equal ranks: the leftmost pair goes first
    assert tok.encode("cba", False) == [v["c"], v["b"], v["a"]]
    tok2 = Tokenizer(spec([("a", "a")]))
    assert tok2.encode("aaa", False) == [tok2.vocab["aa"], tok2.vocab["a"]]


def test_whole_piece_in_vocabulary_wins_when_merges_are_ignored():
    merges = [("a", "b")]
    plain = Tokenizer(spec(merges, extra_vocab=["abc"]))
    whole = Tokenizer(spec(merges, ignore_merges=True, extra_vocab=["abc"]))
    assert plain.encode("abc", False) == [plain.vocab["ab"], plain.vocab["c"]]      # no merge reaches `abc`
    assert whole.encode("abc", False) == [whole.vocab["abc"]]


@pytest.mark.parametrize("text", [
    "the carrier of a contraction is one slot.", "  leading and   inner   runs\n\nand lines\r\n", "it's 1234567 tokens, isn't it?",
    "naïve café — 東京 🙂", "", "\t\x00\x7f"])
def test_round_trip_and_piecewise_structure(text):
    tok = Tokenizer(spec(learn(SAMPLE, 120)))
    ids = tok.encode(text, add_special_tokens=False)
    assert tok.decode(ids) == text
    assert all(0 <= i < len(tok.vocab) for i in ids)
    with_bos = tok.encode(text)                                # encode(prompt, true): the template's begin-of-text token leads
    assert with_bos == [tok.added["<|begin_of_text|>"]] + ids
    assert tok.decode(with_bos) == text and tok.decode(with_bos, skip_special_tokens=False) == "<|begin_of_text|>" + text


def test_learnt_merges_shorten_the_sample_and_special_tokens_are_cut_out():
    tok = Tokenizer(spec(learn(SAMPLE, 120)))
    none = Tokenizer(spec([]))
    assert len(tok.encode(SAMPLE, False)) < len(none.encode(SAMPLE, False)) // 2
    assert len(none.encode("héllo", False)) == 6               # bytes, not characters
    eot = tok.added["<|end_of_text|>"]
    ids = tok.encode("one step<|end_of_text|>next", False)
    assert ids.count(eot) == 1
    cut = ids.index(eot)
    assert ids[:cut] == tok.encode("one step", False) and ids[cut + 1:] == tok.encode("next", False)
    assert tok.decode(ids, skip_special_tokens=False) == "one step<|end_of_text|>next"


def test_refusals_and_file_loading(tmp_path):
    with pytest.raises(TokenizerError, match="only a BPE model"):
        Tokenizer({"model": {"type": "Unigram"}})
    with pytest.raises(TokenizerError, match="no vocabulary"):
        Tokenizer({"model": {"type": "BPE", "vocab": {}}})
    with pytest.raises(TokenizerError, match="load tokenizer"):
        Tokenizer.from_file(str(tmp_path / "absent.json"))
    s = spec(learn(SAMPLE, 40))
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(s), encoding="utf-8")
    tok = Tokenizer.from_file(str(p))
    assert tok.decode(tok.encode("a replay replays")) == "a replay replays"
    with pytest.raises(TokenizerError, match="no token has id"):
        tok.decode([10 ** 6])
    bad = spec([])
    del bad["model"]["vocab"][byte_alphabet()[ord("z")]]
    with pytest.raises(TokenizerError, match="not in the vocabulary"):
        Tokenizer(bad).encode("z", False)
