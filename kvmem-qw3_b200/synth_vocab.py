"""Seeded synthetic inputs for the tokenizer: a byte-level BPE vocabulary trained on seeded pseudo-text, with the irregular
table entries the table-building rules have to cope with.  Stands in for a checkpoint's tokenizer tables (no checkpoint
file is available to this build); used by the tokenizer workload of the benchmark and by the tests."""
import numpy as np


def byte_alphabet():
    """The GPT-2 byte -> visible character table (src/tokenizer.cpp:85-102): printable Latin-1 bytes map to themselves,
    the rest to U+0100, U+0101, ... in byte order."""
    out, nxt = [], 256
    for b in range(256):
        if 0x21 <= b <= 0x7E or 0xA1 <= b <= 0xAC or 0xAE <= b <= 0xFF:
            out.append(chr(b))
        else:
            out.append(chr(nxt))
            nxt += 1
    return out


SPECIAL_TOKENS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>"]


def synth_corpus(seed, n_words=6000):
    """Seeded pseudo-text: Zipf-distributed lower-case words with some capitals, digits, punctuation, CJK and accents."""
    rs = np.random.RandomState(seed & 0x7FFFFFFF)
    letters = "etaoinshrdlcumwfgypbvkjxqz"
    lexicon = ["".join(letters[min(25, int(rs.exponential(6.0)))] for _ in range(1 + int(rs.exponential(3.5)))) for _ in range(400)]
    extra = ["don't", "we'll", "I'm", "it's", "they've", "you're", "he'd", "2024", "3.14", "x=1;", "(a+b)", "{\"k\":[1,2]}", "你好", "世界", "こんにちは",
             "한국어", "café", "naïve", "é", "->", "==", "//", "...", "!?", "#tag", "@me", "$9", "50%", "a_b", "C++"]
    words = []
    for _ in range(n_words):
        r = rs.rand()
        if r < 0.85:
            w = lexicon[min(len(lexicon) - 1, int(rs.zipf(1.3)) - 1)]
            if rs.rand() < 0.1:
                w = w.capitalize()
        else:
            w = extra[rs.randint(len(extra))]
        words.append(w)
    return words


def synth_bpe_vocab(seed, n_merges=700):
    """(tokens, merges) as lists of bytes: 256 byte tokens, the merged symbols in merge order, the special tokens, plus a
    few irregular entries (a duplicate token string, an empty one, a duplicate merge line, a line without a blank) that
    exercise the table-building rules.  Merges come from a plain BPE training pass over synth_corpus()."""
    alpha = byte_alphabet()
    counts = {}
    for w in synth_corpus(seed):
        for form in (w, " " + w):
            sym = tuple(alpha[b] for b in form.encode("utf-8"))
            counts[sym] = counts.get(sym, 0) + 1
    merges, merged_syms = [], []
    words = dict(counts)
    for _ in range(n_merges):
        pairs = {}
        for sym, n in words.items():
            for a, b in zip(sym, sym[1:]):
                pairs[(a, b)] = pairs.get((a, b), 0) + n
        if not pairs:
            break
        (a, b), n = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        if n < 2:
            break
        merges.append(a + " " + b)
        merged_syms.append(a + b)
        nw = {}
        for sym, cnt in words.items():
            out, i = [], 0
            while i < len(sym):
                if i + 1 < len(sym) and sym[i] == a and sym[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(sym[i]); i += 1
            nw[tuple(out)] = nw.get(tuple(out), 0) + cnt
        words = nw
    tokens = list(alpha) + merged_syms + SPECIAL_TOKENS
    tokens += [merged_syms[3], "", "zz_unused"]                  # a repeated string (the first id wins), an empty string
    merges = merges[:50] + [merges[7], "nospaceline"] + merges[50:]   # a repeated line (the first rank wins), a line without a blank
    return [t.encode("utf-8") for t in tokens], [m.encode("utf-8") for m in merges]
