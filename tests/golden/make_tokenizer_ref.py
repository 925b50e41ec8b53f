"""Golden vectors of the reference's tokenizer for the byte-level BPE tokenizer of the product.

The vocabulary is seeded (oracle/gguf_synth.py: synth_bpe_vocab) and so are the texts (texts() below), so only the
RESULTS are stored; they come from the reference's own qw3::QwenTokenizer (encode, decode) and
qw3::detail::qwen_pre_tokenize, called through oracle/_ref/libqw3ref_tokenizer.so (oracle/Makefile target
ref-tokenizer, which links the reference's tokenizer.cpp and gguf.cpp compiled where they lie).  The reference takes
the class of a code point outside its own tables from the process locale; the vectors are made, and compared, under
LC_ALL=C.  Run where the reference tree is present:

    make -C oracle ref-tokenizer REF=<reference tree> && python tests/golden/make_tokenizer_ref.py

Writes tests/golden/tokenizer_ref.npz: per text the token ids (without and with BOS), the piece ends of the text between
special tokens being left to the encoder, and the bytes the reference decodes the ids back to.
"""
import ctypes
import os
import sys
import tempfile

os.environ["LC_ALL"] = "C"

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "tokenizer_ref.npz")
VOCAB_SEED = 0x70C


def texts():
    """Seeded list of byte strings: hand-written edge cases, then random mixtures of word-like, numeric, symbolic, blank,
    CJK, accented, combining, 4-byte and malformed pieces with special tokens strewn in."""
    fixed = [
        b"", b" ", b"  ", b"\n", b"\r\n", b" \n ", b"a", b" a", b"  a", b"a ", b"a  ", b"a\n", b"a \n b", b"\t\ta", b"a\t\tb",
        b"Hello, world!", b"Hello,  world!  ", b"don't DON'T it's I'M we'll WE'LL they've you're he'd 'RE 're' 'x", b"'", b"''", b"'s", b"x's'", b"'l", b"'ll",
        b"1", b"12", b"123", b"3.14159", b" 42", b"  42", b"a1b2", b"1a", b"v2.0-rc1", b"0x7F", b"1,000,000", b"2024-11-25T12:34:56Z",
        b"x=1;", b"(a+b)*c", b" (alpha)", b"a  +  b", b"{\"k\": [1, 2, 3], \"s\": \"t\"}", b"if (x) {\n    return y;\n}\n", b"def f(a, b):\n\treturn a+b\n",
        b"...", b" ...", b"!?!?", b"a...b", b"end.\n\nNext", b"end.\r\n\r\nNext", b"#tag @me $9 50% a_b C++ ->  ==  //",
        "你好世界".encode(), " 你好 世界 ".encode(), "こんにちは、世界。".encode(), "한국어 텍스트".encode(), "abc你好def".encode(), "１２３ ＡＢＣ".encode(),
        "café naïve résumé".encode(), "é".encode(), " é".encode(), "aé".encode(), "Ωμέγα".encode(), "é".encode(), "à́b".encode(), "́".encode(), " ́x".encode(),
        "a b".encode(), "a  b".encode(), "a b".encode(), "a　b".encode(), "a\u0085b".encode(), "😀".encode(), "hi 😀 there".encode(), "😀😀".encode(),
        b"\xff", b"a\xffb", b"\xc3", b"ab\xc3", b"\xe4\xbd", b"\xf0\x9f\x98", b"\x80\x80", b"\xc0\x80", b"\x00", b"a\x00b", b"\x7f\x01\x1f",
        b"<|im_start|>", b"<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n", b"<think>\n\n</think>\n\nOK", b"<|im_start|><|im_end|>", b"a<|endoftext|>b",
        b"<|im_start", b"<|im_start|", b"<think", b"<", b"<<|im_end|>>", b"<|im_end|><", b"<tool_call>{\"name\": \"f\"}</tool_call>", b"<|fim_prefix|>x", b"< |im_end|>",
        b"</think >", b"<|IM_START|>", b"  <think>  ",
    ]
    g = np.random.default_rng(0x70CE)
    letters = "etaoinshrdlcumwfgypbvkjxqzETAOIN"
    parts = {
        "word": lambda: "".join(letters[int(g.integers(len(letters)))] for _ in range(int(g.integers(1, 9)))).encode(),
        "num": lambda: str(int(g.integers(0, 100000))).encode(),
        "sym": lambda: "".join("!\"#$%&()*+,-./:;<=>?@[\\]^_`{|}~'"[int(g.integers(32))] for _ in range(int(g.integers(1, 4)))).encode(),
        "blank": lambda: "".join(" \t\n\r\v\f"[int(g.choice([0, 0, 0, 0, 1, 2, 2, 3, 4, 5]))] for _ in range(int(g.integers(1, 5)))).encode(),
        "cjk": lambda: "".join(chr(int(g.integers(0x4E00, 0x9FFF))) for _ in range(int(g.integers(1, 4)))).encode(),
        "kana": lambda: "".join(chr(int(g.integers(0x3041, 0x30FF))) for _ in range(int(g.integers(1, 4)))).encode(),
        "latin1": lambda: "".join(chr(int(g.integers(0xC0, 0xFF))) for _ in range(int(g.integers(1, 3)))).encode(),
        "mark": lambda: chr(int(g.integers(0x0300, 0x036F))).encode(),
        "uspace": lambda: chr(int(g.choice([0xA0, 0x2002, 0x2009, 0x2028, 0x2029, 0x3000, 0x205F]))).encode(),
        "wide": lambda: chr(int(g.integers(0x1F600, 0x1F64F))).encode(),
        "junk": lambda: bytes(int(g.integers(0x80, 0x100)) for _ in range(int(g.integers(1, 3)))),
        "quote": lambda: [b"'s", b"'T", b"'re", b"'VE", b"'m", b"'ll", b"'d", b"'x", b"'"][int(g.integers(9))],
        "special": lambda: [b"<|im_start|>", b"<|im_end|>", b"<|endoftext|>", b"<think>", b"</think>", b"<tool_call>", b"</tool_call>", b"<|im_", b"<thin"][int(g.integers(9))],
    }
    kinds = list(parts)
    weights = np.array([10, 3, 4, 8, 2, 1, 1, 1, 1, 1, 1, 2, 1.5], np.float64)
    weights /= weights.sum()
    rnd = []
    for _ in range(320):
        n = int(g.integers(1, 40))
        rnd.append(b"".join(parts[kinds[int(g.choice(len(kinds), p=weights))]]() for _ in range(n)))
    return fixed + rnd


def blob(items):
    offs = np.zeros(len(items) + 1, np.int64)
    for i, x in enumerate(items):
        offs[i + 1] = offs[i] + len(x)
    return np.frombuffer(b"".join(items), np.uint8).copy(), offs


def main():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import gguf_synth as G
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libqw3ref_tokenizer.so"))
    L.rt_open.restype = ctypes.c_void_p
    L.rt_open.argtypes = [ctypes.c_char_p]
    L.rt_encode.restype = ctypes.c_int64
    L.rt_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64]
    L.rt_decode.restype = ctypes.c_int64
    L.rt_decode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64]
    L.rt_split.restype = ctypes.c_int64
    L.rt_split.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64]
    tokens, merges = G.synth_bpe_vocab(VOCAB_SEED)
    bos = tokens.index(b"<|endoftext|>")
    eos = tokens.index(b"<|im_end|>")
    with tempfile.TemporaryDirectory() as d:
        h = L.rt_open(G.write_tokenizer_gguf(os.path.join(d, "tok.gguf"), tokens, merges, bos, eos, False).encode())
        assert h, "the reference could not read the synthetic tokenizer file"
        ids_all, ids_off, bos_first, ends_all, ends_off, dec = [], [0], [], [], [0], []
        for t in texts():
            cap = len(t) + 8
            ids = np.zeros(cap, np.int32)
            n = L.rt_encode(h, t, len(t), 0, ids.ctypes.data, cap)
            assert n <= cap
            wb = np.zeros(cap, np.int32)
            nb = L.rt_encode(h, t, len(t), 1, wb.ctypes.data, cap)
            assert nb == n + 1 and np.array_equal(wb[1:nb], ids[:n])
            bos_first.append(int(wb[0]))
            ids_all.append(ids[:n].copy())
            ids_off.append(ids_off[-1] + n)
            ends = np.zeros(cap, np.uint32)
            ne = L.rt_split(t, len(t), ends.ctypes.data, cap)
            assert ne <= cap
            ends_all.append(ends[:ne].copy())
            ends_off.append(ends_off[-1] + ne)
            buf = ctypes.create_string_buffer(8 * cap + 64)
            nd = L.rt_decode(h, ids.ctypes.data, n, buf, len(buf))
            assert nd <= len(buf)
            dec.append(buf.raw[:nd])
    dec_blob, dec_off = blob(dec)
    np.savez_compressed(OUT, vocab_seed=VOCAB_SEED, n_texts=len(dec), bos_id=bos, eos_id=eos, bos_first=np.array(bos_first, np.int32),
                        ids=np.concatenate(ids_all).astype(np.int32), ids_off=np.array(ids_off, np.int64),
                        ends=np.concatenate(ends_all).astype(np.uint32), ends_off=np.array(ends_off, np.int64), dec=dec_blob, dec_off=dec_off)
    print("wrote", OUT, ":", len(dec), "texts,", ids_off[-1], "tokens,", ends_off[-1], "pieces")


if __name__ == "__main__":
    main()
