"""The byte-level BPE tokenizer (host only) against the reference's own: golden vectors made by qw3::QwenTokenizer and
qw3::detail::qwen_pre_tokenize on a seeded vocabulary and 421 seeded texts (tests/golden/make_tokenizer_ref.py), the ten
known answers of the reference's tests/tokenizer_pretokenizer_test.cpp, and, where the reference's tokenizer has been
built (oracle/_ref/libqw3ref_tokenizer.so), fresh random texts through both."""
import ctypes
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import gguf_synth as G  # noqa: E402
import make_tokenizer_ref as M  # noqa: E402

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libqw3ref_tokenizer.so")


@pytest.fixture(scope="module")
def vocab():
    tokens, merges = G.synth_bpe_vocab(M.VOCAB_SEED)
    return tokens, merges, tokens.index(b"<|endoftext|>"), tokens.index(b"<|im_end|>")


@pytest.fixture(scope="module")
def tok(qb, vocab):
    tokens, merges, bos, eos = vocab
    t = qb.binding.Tokenizer.from_tables(tokens, merges, bos, eos, False)
    yield t
    t.close()


def test_tables_follow_the_reference_rules(tok, vocab):
    tokens, merges, bos, eos = vocab
    assert tok.vocab_size == len(tokens) and tok.bos_id == bos and tok.eos_id == eos and not tok.add_bos_default
    assert tok.n_special == len(G.SPECIAL_TOKENS)
    dup = tokens[-3]                                        # the repeated string keeps its first id
    assert tokens.count(dup) == 2 and tok.token_id(dup) == tokens.index(dup)
    assert tok.token_id(b"") == -1 and tok.token_id(b"no such token") == -1
    assert tok.token_id(b"<think>") == tokens.index(b"<think>")


def test_known_answers_of_the_reference_pretokenizer_test(qb):
    split = qb.binding.Tokenizer.split
    cases = [(" alpha", [" alpha"]), ("  alpha", [" ", " alpha"]), ("    alpha", ["   ", " alpha"]), ("    20", ["   ", " ", "2", "0"]),
             (" (alpha)", [" (", "alpha", ")"]), ("a  +  b", ["a", " ", " +", " ", " b"]), ("\t\talpha", ["\t", "\talpha"]),
             ("alpha\n    beta", ["alpha", "\n", "   ", " beta"]), ("123", ["1", "2", "3"]), ("'RE", ["'RE"])]
    for text, want in cases:
        assert [p.decode() for p in split(text)] == want, text


def test_golden_vectors_of_the_reference(qb, tok):
    g = np.load(os.path.join(HERE, "golden", "tokenizer_ref.npz"))
    texts = M.texts()
    assert int(g["vocab_seed"]) == M.VOCAB_SEED and int(g["n_texts"]) == len(texts)
    n_tok = n_piece = 0
    for i, t in enumerate(texts):
        want = g["ids"][g["ids_off"][i]:g["ids_off"][i + 1]]
        got = tok.encode(t)
        assert np.array_equal(got, want), (i, t, got.tolist(), want.tolist())
        with_bos = tok.encode(t, add_bos=True)
        assert with_bos[0] == g["bos_first"][i] == tok.bos_id and np.array_equal(with_bos[1:], want)
        ends = g["ends"][g["ends_off"][i]:g["ends_off"][i + 1]].tolist()
        pieces = qb.binding.Tokenizer.split(t)
        assert np.cumsum([len(p) for p in pieces]).tolist() == ends, (i, t, pieces)
        dec = bytes(g["dec"][g["dec_off"][i]:g["dec_off"][i + 1]])
        assert tok.decode(want) == dec == t, (i, t)         # every byte and every special token is in the vocabulary
        n_tok += len(want)
        n_piece += len(ends)
    print("tokenizer golden vectors: %d texts, %d tokens, %d pieces equal to the reference's" % (len(texts), n_tok, n_piece))


def test_file_and_tables_build_the_same_tokenizer(qb, tok, vocab, tmp_path):
    tokens, merges, bos, eos = vocab
    path = G.write_tokenizer_gguf(str(tmp_path / "tok.gguf"), tokens, merges, bos, eos, True)
    f = qb.binding.Tokenizer.from_gguf(path)
    assert (f.vocab_size, f.bos_id, f.eos_id, f.add_bos_default, f.n_special) == (tok.vocab_size, bos, eos, True, tok.n_special)
    for t in M.texts()[::7]:
        ids = f.encode(t)                                   # the checkpoint asks for BOS by default
        assert ids[0] == bos and np.array_equal(ids[1:], tok.encode(t))
    f.close()
    bad = G.write_tokenizer_gguf(str(tmp_path / "bad.gguf"), tokens, merges, bos, eos, False)
    raw = open(bad, "rb").read().replace(b"tokenizer.ggml.merges", b"tokenizer.ggml.merged")
    open(bad, "wb").write(raw)
    with pytest.raises(qb.binding.QbError, match="merges"):
        qb.binding.Tokenizer.from_gguf(bad)


def test_damaged_files_are_refused(qb, vocab, tmp_path):
    tokens, merges, bos, eos = vocab
    good = G.write_tokenizer_gguf(str(tmp_path / "tok.gguf"), tokens, merges, bos, eos, False)
    raw = open(good, "rb").read()
    for cut in (0, 3, 20, 24, 200, len(raw) // 2, len(raw) - 40):      # truncations inside the header, a key, a string array
        bad = str(tmp_path / ("cut%d.gguf" % cut))
        open(bad, "wb").write(raw[:cut])
        with pytest.raises(qb.binding.QbError):
            qb.binding.Tokenizer.from_gguf(bad)
    huge = bytearray(raw)
    at = raw.index(b"tokenizer.ggml.tokens") + len(b"tokenizer.ggml.tokens") + 4 + 4      # the array's element count
    huge[at:at + 8] = (2 ** 62).to_bytes(8, "little")
    bad = str(tmp_path / "count.gguf")
    open(bad, "wb").write(bytes(huge))
    with pytest.raises(qb.binding.QbError):
        qb.binding.Tokenizer.from_gguf(bad)
    with pytest.raises(qb.binding.QbError):
        qb.binding.Tokenizer.from_gguf(str(tmp_path / "missing.gguf"))


def test_capacity_is_reported_not_overrun(qb, tok):
    L = qb.lib()
    text = b"one two three four five"
    n = ctypes.c_size_t()
    ids = np.full(4, -7, np.int32)
    st = L.qb_tokenizer_encode(tok.h, text, len(text), 0, ids.ctypes.data, 2, ctypes.byref(n))
    assert st != 0 and n.value == len(tok.encode(text)) > 2 and ids.tolist() == [-7] * 4
    out = ctypes.create_string_buffer(4)
    full = tok.encode(text)
    st = L.qb_tokenizer_decode(tok.h, full.ctypes.data, full.size, out, 4, ctypes.byref(n))
    assert st != 0 and n.value == len(text)
    assert tok.decode(np.array([-1, tok.vocab_size, 10 ** 6], np.int32)) == b""


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="the reference's tokenizer is not built here (make -C oracle ref-tokenizer)")
def test_fresh_random_texts_through_both_tokenizers(qb, tok, vocab, tmp_path):
    tokens, merges, bos, eos = vocab
    L = ctypes.CDLL(REF_LIB)
    L.rt_open.restype = ctypes.c_void_p
    L.rt_open.argtypes = [ctypes.c_char_p]
    L.rt_encode.restype = ctypes.c_int64
    L.rt_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64]
    L.rt_split.restype = ctypes.c_int64
    L.rt_split.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64]
    h = L.rt_open(G.write_tokenizer_gguf(str(tmp_path / "tok.gguf"), tokens, merges, bos, eos, False).encode())
    assert h
    g = np.random.default_rng(0xF2E5)
    base = [t for t in M.texts() if t]
    total = 0
    for _ in range(300):
        # splice pieces of the seeded texts at random byte positions: new boundaries, new malformed sequences
        parts = []
        for _ in range(int(g.integers(1, 6))):
            t = base[int(g.integers(len(base)))]
            a = int(g.integers(0, len(t)))
            parts.append(t[a:a + int(g.integers(1, 40))])
        t = b"".join(parts)
        cap = len(t) + 8
        ids = np.zeros(cap, np.int32)
        n = L.rt_encode(h, t, len(t), 0, ids.ctypes.data, cap)
        assert np.array_equal(tok.encode(t), ids[:n]), t
        ends = np.zeros(cap, np.uint32)
        ne = L.rt_split(t, len(t), ends.ctypes.data, cap)
        assert np.cumsum([len(p) for p in qb.binding.Tokenizer.split(t)]).tolist() == ends[:ne].tolist(), t
        total += n
    L.rt_close.argtypes = [ctypes.c_void_p]
    L.rt_close(h)
    print("tokenizer against the reference's, 300 spliced texts: %d tokens equal" % total)
