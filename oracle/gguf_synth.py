"""Seeded synthetic qwen35 checkpoints as named tensors and as GGUF v3 files.

TEST INFRASTRUCTURE ONLY (used by tests/ and by the reference-executor comparator under oracle/): the same
tensors feed the product (`qb_model_create` / `qb_model_load_gguf`), the CPU oracle
(`orc_model_create_tensors`) and, through the file, the reference's own GGUF reader (src/gguf.cpp:216-278;
tensor names src/qwen_native.cpp:147-190 and :271-298; metadata keys src/qwen_config.cpp:53-108; only the
tensor types F32 = 0 and Q8_0 = 8, src/model_source.cpp:120-121).

Unlike the seeded model of the benchmark (all RMSNorm gains 1.0), the gains here are 1 + gain_sigma * N(0,1),
every norm with its own draws, so that a mixed-up gain vector (enorm / hnorm, attn_norm / ffn_norm, q / k
norm) changes the result.
"""
import struct

import numpy as np

import oracle as O

GGUF_MAGIC = 0x46554747
T_U32, T_F32, T_BOOL, T_STR, T_ARR = 4, 6, 7, 8, 9


def _q8(seed, tid, rows, cols, sigma):
    return O.synth_q8_0(seed, tid, rows, cols, sigma).reshape(rows, cols // 32 * 34)


def synth_tensors(cfg, seed, gain_sigma=0.1, sigma=0.02, own_mtp_tables=False):
    """{GGUF tensor name: numpy array} of a whole model: uint8 [rows][cols/32*34] for Q8_0, float32 for F32.
    Layer i is full attention iff (i + 1) % full_attention_interval == 0; the MTP layer is block n_layers."""
    c = cfg
    rs = np.random.RandomState(seed & 0x7FFFFFFF)
    H, F, V = c.n_embd, c.n_ff, c.vocab_size
    inner, kvd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
    nk, nv, hd = c.ssm_num_k_heads, c.ssm_num_v_heads, c.ssm_head_dim
    C_, vdim = (2 * nk + nv) * hd, nv * hd
    t, tid = {}, [0]

    def q8(name, rows, cols):
        tid[0] += 1
        t[name] = _q8(seed, 0x100000 + tid[0], rows, cols, sigma)

    def gain(name, n):
        t[name] = (1.0 + gain_sigma * rs.randn(n)).astype(np.float32)

    def layer(il, attn):
        b = "blk.%d." % il
        gain(b + "attn_norm.weight", H)
        gain(b + "post_attention_norm.weight", H)
        if attn:
            q8(b + "attn_q.weight", 2 * inner, H); q8(b + "attn_k.weight", kvd, H); q8(b + "attn_v.weight", kvd, H)
            q8(b + "attn_output.weight", H, inner)
            gain(b + "attn_q_norm.weight", c.head_dim); gain(b + "attn_k_norm.weight", c.head_dim)
        else:
            q8(b + "attn_qkv.weight", C_, H); q8(b + "attn_gate.weight", vdim, H)
            q8(b + "ssm_alpha.weight", nv, H); q8(b + "ssm_beta.weight", nv, H); q8(b + "ssm_out.weight", H, vdim)
            t[b + "ssm_conv1d.weight"] = ((rs.rand(C_, c.ssm_conv_kernel) * 2 - 1) * 0.5).astype(np.float32)
            t[b + "ssm_a"] = (-np.exp(rs.rand(nv) * np.log(16.0))).astype(np.float32)
            t[b + "ssm_dt.bias"] = (-4.0 + 3.0 * rs.rand(nv)).astype(np.float32)
            gain(b + "ssm_norm.weight", hd)
        q8(b + "ffn_gate.weight", F, H); q8(b + "ffn_up.weight", F, H); q8(b + "ffn_down.weight", H, F)

    q8("token_embd.weight", V, H)
    q8("output.weight", V, H)
    gain("output_norm.weight", H)
    for il in range(c.n_layers):
        layer(il, c.full_attention_interval and (il + 1) % c.full_attention_interval == 0)
    if c.mtp_layers:
        il = c.n_layers
        layer(il, True)
        b = "blk.%d.nextn." % il
        q8(b + "eh_proj.weight", H, 2 * H)
        gain(b + "enorm.weight", H); gain(b + "hnorm.weight", H); gain(b + "shared_head_norm.weight", H)
        if own_mtp_tables:
            q8(b + "embed_tokens.weight", V, H); q8(b + "shared_head_head.weight", V, H)
    return t


# Tensor ids of the seeded benchmark model: layer * 32 + kind, globals under layer 0xFFFF (the enum of the engine
# and of the oracle's build_layer).
(K_ATTN_Q, K_ATTN_K, K_ATTN_V, K_ATTN_OUT, K_FFN_GATE, K_FFN_UP, K_FFN_DOWN, K_SSM_QKV, K_SSM_Z, K_SSM_ALPHA, K_SSM_BETA,
 K_SSM_OUT, K_SSM_CONV, K_SSM_A, K_SSM_DT, K_EH_PROJ, K_TOKEN_EMBD, K_OUTPUT) = range(1, 19)


def seeded_model_tensors(cfg, seed, gain_sigma=0.0, gain_seed=77, branch_scale=1.0, eh_identity=False):
    """The seeded random-init model of the benchmark (qb_model_create_synth / orc_model_create: every Q8_0 tensor
    quantise(N(0, sigma^2)) from the counter-based generator, ssm_a = -exp(U(0, ln 16)), dt_bias ~ U(-4, -1),
    conv1d ~ U(-0.5, 0.5)) as named tensors.  gain_sigma = 0 keeps its unit RMSNorm gains (then the model built
    from these tensors equals the seeded one bit for bit); > 0 draws every gain as 1 + gain_sigma * N(0, 1).

    branch_scale < 1 and eh_identity make a model whose MTP head has a real acceptance rate without training: the
    projections that write into the residual stream (attn_output, ssm_out, ffn_down) are scaled down, so the next
    token depends mostly on the current token's embedding, and eh_proj is [I | 0] plus the seeded noise, so the MTP
    head sees that embedding too.  Every layer still contributes: how often a draft is accepted then depends on the
    whole wiring of the head (its K/V prefix, the hidden row it is fed, the positions)."""
    c = cfg
    H, F, V, sg = c.n_embd, c.n_ff, c.vocab_size, c.weight_sigma
    inner, kvd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
    nk, nv, hd = c.ssm_num_k_heads, c.ssm_num_v_heads, c.ssm_head_dim
    C_, vdim = (2 * nk + nv) * hd, nv * hd
    rs = np.random.RandomState(gain_seed)
    t = {}
    tid = lambda il, kind: il * 32 + kind
    BRANCH = (K_ATTN_OUT, K_SSM_OUT, K_FFN_DOWN)
    q8 = lambda name, il, kind, rows, cols: t.__setitem__(name, _q8(seed, tid(il, kind), rows, cols, sg * (branch_scale if kind in BRANCH else 1.0)))
    u = lambda il, kind, n: (O.rand_u32(seed, tid(il, kind), n) >> 8).astype(np.float64) / 16777216.0

    def gain(name, n):
        t[name] = (1.0 + gain_sigma * rs.randn(n)).astype(np.float32) if gain_sigma else np.ones(n, np.float32)

    def layer(il, attn):
        b = "blk.%d." % il
        gain(b + "attn_norm.weight", H); gain(b + "ffn_norm.weight", H)
        if attn:
            q8(b + "attn_q.weight", il, K_ATTN_Q, 2 * inner, H); q8(b + "attn_k.weight", il, K_ATTN_K, kvd, H)
            q8(b + "attn_v.weight", il, K_ATTN_V, kvd, H); q8(b + "attn_output.weight", il, K_ATTN_OUT, H, inner)
            gain(b + "attn_q_norm.weight", c.head_dim); gain(b + "attn_k_norm.weight", c.head_dim)
        else:
            q8(b + "attn_qkv.weight", il, K_SSM_QKV, C_, H); q8(b + "attn_gate.weight", il, K_SSM_Z, vdim, H)
            q8(b + "ssm_alpha.weight", il, K_SSM_ALPHA, nv, H); q8(b + "ssm_beta.weight", il, K_SSM_BETA, nv, H)
            q8(b + "ssm_out.weight", il, K_SSM_OUT, H, vdim)
            t[b + "ssm_conv1d.weight"] = ((u(il, K_SSM_CONV, C_ * c.ssm_conv_kernel) * 2.0 - 1.0) * 0.5).astype(np.float32).reshape(C_, c.ssm_conv_kernel)
            t[b + "ssm_a"] = (-np.exp(u(il, K_SSM_A, nv) * np.log(16.0))).astype(np.float32)
            t[b + "ssm_dt.bias"] = (-4.0 + 3.0 * u(il, K_SSM_DT, nv)).astype(np.float32)
            gain(b + "ssm_norm.weight", hd)
        q8(b + "ffn_gate.weight", il, K_FFN_GATE, F, H); q8(b + "ffn_up.weight", il, K_FFN_UP, F, H)
        q8(b + "ffn_down.weight", il, K_FFN_DOWN, H, F)

    q8("token_embd.weight", 0xFFFF, K_TOKEN_EMBD, V, H)
    q8("output.weight", 0xFFFF, K_OUTPUT, V, H)
    gain("output_norm.weight", H)
    for il in range(c.n_layers):
        layer(il, bool(c.full_attention_interval) and (il + 1) % c.full_attention_interval == 0)
    if c.mtp_layers:
        il = c.n_layers
        layer(il, True)
        b = "blk.%d.nextn." % il
        q8(b + "eh_proj.weight", il, K_EH_PROJ, H, 2 * H)
        if eh_identity:
            w = O.dequant_q8_0(t[b + "eh_proj.weight"].reshape(-1), H, 2 * H) * branch_scale
            w[np.arange(H), np.arange(H)] += 1.0
            t[b + "eh_proj.weight"] = O.quantize_q8_0(w).reshape(H, 2 * H // 32 * 34)
        gain(b + "enorm.weight", H); gain(b + "hnorm.weight", H); gain(b + "shared_head_norm.weight", H)
    return t


def token_strings(vocab):
    """One printable ASCII string per token id, fixed width, so that text produced by the reference's tokenizer
    (byte-level decode, src/tokenizer.cpp:719-745) splits back into token ids: 't' + 7 digits + ';'."""
    return ["t%07d;" % i for i in range(vocab)]


def parse_token_text(text):
    assert len(text) % 9 == 0, "text is not a concatenation of synthetic token strings"
    out = []
    for i in range(0, len(text), 9):
        piece = text[i:i + 9]
        assert piece[0] == "t" and piece[8] == ";", piece
        out.append(int(piece[1:8]))
    return out


def _s(b):
    b = b.encode() if isinstance(b, str) else b
    return struct.pack("<Q", len(b)) + b


def _kv(key, typ, payload):
    return _s(key) + struct.pack("<I", typ) + payload


def write_gguf(path, cfg, tensors, context_length=4096, eos_id=None, tokens=None, merges=None):
    """GGUF v3, alignment 32, metadata of a qwen35 checkpoint, tensors in dict order.  tokens / merges: the tokenizer's
    tables (bytes; default: the fixed-width synthetic token strings and no merges); a shorter token table is filled up
    to the vocabulary size with unused names."""
    c, p = cfg, "qwen35."
    toks = token_strings(c.vocab_size) if tokens is None else list(tokens) + [b"<unused%d>" % i for i in range(len(tokens), c.vocab_size)]
    assert len(toks) == c.vocab_size
    u32 = lambda k, v: _kv(k, T_U32, struct.pack("<I", int(v)))
    f32 = lambda k, v: _kv(k, T_F32, struct.pack("<f", float(v)))
    strs = lambda k, a: _kv(k, T_ARR, struct.pack("<IQ", T_STR, len(a)) + b"".join(_s(x) for x in a))
    kv = [
        _kv("general.architecture", T_STR, _s("qwen35")),
        u32("general.alignment", 32),
        u32(p + "block_count", c.n_layers + c.mtp_layers), u32(p + "nextn_predict_layers", c.mtp_layers),
        u32(p + "embedding_length", c.n_embd), u32(p + "feed_forward_length", c.n_ff), u32(p + "context_length", context_length),
        u32(p + "attention.head_count", c.n_heads), u32(p + "attention.head_count_kv", c.n_kv_heads),
        u32(p + "attention.key_length", c.head_dim), u32(p + "attention.value_length", c.head_dim),
        f32(p + "attention.layer_norm_rms_epsilon", c.rms_eps),
        u32(p + "rope.dimension_count", c.rope_dim), f32(p + "rope.freq_base", c.rope_theta),
        u32(p + "ssm.conv_kernel", c.ssm_conv_kernel), u32(p + "ssm.state_size", c.ssm_head_dim),
        u32(p + "ssm.time_step_rank", c.ssm_num_v_heads), u32(p + "ssm.group_count", c.ssm_num_k_heads),
        u32(p + "ssm.inner_size", (2 * c.ssm_num_k_heads + c.ssm_num_v_heads) * c.ssm_head_dim),
        u32(p + "full_attention_interval", c.full_attention_interval),
        _kv("tokenizer.ggml.model", T_STR, _s("gpt2")),
        strs("tokenizer.ggml.tokens", toks), strs("tokenizer.ggml.merges", [] if merges is None else list(merges)),
        u32("tokenizer.ggml.bos_token_id", 0), u32("tokenizer.ggml.eos_token_id", c.vocab_size - 1 if eos_id is None else eos_id),
        _kv("tokenizer.ggml.add_bos_token", T_BOOL, struct.pack("<B", 0)),
    ]
    infos, off, blobs = [], 0, []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint8:                                     # Q8_0 rows
            rows, cols, typ = a.shape[0], a.shape[1] // 34 * 32, 8
            dims = [cols, rows]
        else:
            assert a.dtype == np.float32, name
            typ, dims = 0, list(a.shape[::-1])
        infos.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, off))
        blobs.append((off, a))
        off = (off + a.nbytes + 31) // 32 * 32
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    pad = (-len(head)) % 32
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        base = f.tell()
        for o, a in blobs:
            f.seek(base + o)
            f.write(a.tobytes())
        f.truncate(base + off)
    return path


# ---- the seeded byte-level BPE vocabulary of the tokenizer tests: kept with the product's other seeded inputs ------

def _vocab_module():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "kvmem-qw3_b200", "synth_vocab.py")
    spec = importlib.util.spec_from_file_location("qw3b200_synth_vocab", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_V = _vocab_module()
byte_alphabet, SPECIAL_TOKENS, synth_corpus, synth_bpe_vocab = _V.byte_alphabet, _V.SPECIAL_TOKENS, _V.synth_corpus, _V.synth_bpe_vocab


def write_tokenizer_gguf(path, tokens, merges, bos_id, eos_id, add_bos):
    """A GGUF v3 file that holds only what the tokenizer reads (no tensors)."""
    u32 = lambda k, v: _kv(k, T_U32, struct.pack("<I", int(v)))
    strs = lambda k, a: _kv(k, T_ARR, struct.pack("<IQ", T_STR, len(a)) + b"".join(_s(x) for x in a))
    kv = [
        _kv("general.architecture", T_STR, _s("qwen35")), u32("general.alignment", 32),
        _kv("tokenizer.ggml.model", T_STR, _s("gpt2")),
        strs("tokenizer.ggml.tokens", tokens), strs("tokenizer.ggml.merges", merges),
        u32("tokenizer.ggml.bos_token_id", bos_id), u32("tokenizer.ggml.eos_token_id", eos_id),
        _kv("tokenizer.ggml.add_bos_token", T_BOOL, struct.pack("<B", 1 if add_bos else 0)),
    ]
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, 0, len(kv)) + b"".join(kv)
    with open(path, "wb") as f:
        f.write(head + b"\0" * ((-len(head)) % 32))
    return path
