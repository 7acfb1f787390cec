"""CPU-only: the tokenizer boundary (gt_init / gt_encode / gt_encode_mt / gt_decode / gt_free of libbunker_tok.so) against
a plain-Python byte-level BPE that pre-tokenizes with the Qwen regular expression itself."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import regex

from bunker_b200 import tokenizer as T

QWEN_PAT = regex.compile(r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")


def byte_table():
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def make_tokenizer_json(path, corpus: str, n_merges: int = 300):
    """Learn a small BPE on `corpus` (greedy most-frequent-pair merges) and write it in the Hugging Face layout."""
    bt = byte_table()
    words = [[bt[b] for b in w.encode()] for w in QWEN_PAT.findall(corpus)]
    vocab = {bt[b]: i for i, b in enumerate(range(256))}
    merges = []
    for _ in range(n_merges):
        cnt = {}
        for w in words:
            for a, b in zip(w, w[1:]):
                cnt[(a, b)] = cnt.get((a, b), 0) + 1
        if not cnt:
            break
        (a, b), c = max(cnt.items(), key=lambda kv: (kv[1], kv[0]))
        if c < 2:
            break
        merges.append((a, b))
        vocab[a + b] = len(vocab)
        for w in words:
            i = 0
            while i + 1 < len(w):
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [a + b]
                else:
                    i += 1
    added = [{"id": len(vocab), "content": "<|endoftext|>", "special": True},
             {"id": len(vocab) + 1, "content": "<|im_start|>", "special": True}]
    js = {"version": "1.0", "added_tokens": added,
          "model": {"type": "BPE", "vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]}}
    with open(path, "w", encoding="utf-8") as f:
        json.dump(js, f, ensure_ascii=True)     # non-ASCII symbols travel as \\uXXXX escapes
    return vocab, merges, {a["content"]: a["id"] for a in added}


def py_encode(text: str, vocab, merges, added):
    rank = {m: i for i, m in enumerate(merges)}
    bt = byte_table()
    out = []
    pieces = regex.split("(" + "|".join(regex.escape(a) for a in sorted(added, key=len, reverse=True)) + ")", text)
    for piece in pieces:
        if piece in added:
            out.append(added[piece])
            continue
        for w in QWEN_PAT.findall(piece):
            sym = [bt[b] for b in w.encode()]
            while len(sym) > 1:
                best = min(((rank.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(sym, sym[1:]))))
                if best[0] == 1 << 30:
                    break
                i = best[1]
                sym[i:i + 2] = [sym[i] + sym[i + 1]]
            out += [vocab[s] for s in sym]
    return out


CORPUS = ("Hello world, hello there!  The quick brown fox jumps over the lazy dog. It's 12345 o'clock, we're done.\n"
          "def f(x):\n    return x * 2  # double\n\n\nPrices: $3.50, 10% off -- \"quoted\" text; tabs\there.\r\n"
          "Привет мир, こんにちは世界, naïve café über straße. ") * 3

TEXTS = ["Hello world", "hello  world   with   spaces ", "It's we're I'LL don't 'tis", "a1b22c333 4", "x=3;y=4 // c\n\n  next",
         "  leading and trailing  \n", "tab\tsep\t\tdouble", "Привет, мир! こんにちは 世界。", "naïve café", "<|im_start|>user\nhi<|endoftext|>",
         "mix<|endoftext|><|endoftext|>end", "", " ", "\n", "!!!???...\n\nnew", "price $3.50 (10% off)", "line1\r\nline2\rline3"]


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    p = os.path.join(tmp_path_factory.mktemp("tok"), "tokenizer.json")
    vocab, merges, added = make_tokenizer_json(p, CORPUS)
    t = T.Tokenizer(p)
    yield t, vocab, merges, added
    t.close()


def test_library_exports_the_reference_entry_points():
    lib = T.load_library()
    for name in ("gt_init", "gt_encode", "gt_encode_mt", "gt_decode", "gt_vocab_size", "gt_free"):
        assert hasattr(lib, name), name
    assert lib.gt_init(b"/nonexistent/tokenizer.json") is None
    assert lib.gt_encode(None, b"x", 1, (C.c_uint32 * 4)(), 4) == -1


@pytest.mark.parametrize("text", TEXTS)
def test_encode_matches_python_bpe_and_round_trips(tok, text):
    t, vocab, merges, added = tok
    got = t.encode(text)
    want = py_encode(text, vocab, merges, added)
    assert list(got) == want, (text, list(got), want)
    assert t.decode(got) == text
    assert t.vocab_size == len(vocab) + len(added)


def test_multithreaded_encode_keeps_text_order(tok):
    t, vocab, merges, added = tok
    text = CORPUS * 400                      # large enough to be cut into chunks on any core count
    one = t.encode(text)
    many = t.encode(text, threads=True)
    assert len(one) > 50000
    assert t.decode(many) == text            # chunk boundaries may tokenize a space differently, the text is the same
    assert abs(len(many) - len(one)) < 512
    # the out_max contract of the reference: never more ids written than the caller's buffer holds
    lib = T.load_library()
    small = (C.c_uint32 * 8)()
    raw = b"Hello world, hello there!"
    assert lib.gt_encode(t.h, raw, len(raw), small, 3) == 3
    assert list(small[:3]) == list(t.encode(raw.decode())[:3])
