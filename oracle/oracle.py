"""ctypes wrapper of the CPU oracle (oracle/qw3_oracle.cpp).

Test infrastructure only: imported by tests/, by the smoke entry and by the CPU-baseline leg of
bench.py, never by the product package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class ModelConfig(C.Structure):
    """Mirror of qb_model_config (include/qw3b200.h)."""
    _fields_ = [
        ("n_layers", C.c_uint32), ("n_embd", C.c_uint32), ("n_ff", C.c_uint32),
        ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("rope_dim", C.c_uint32), ("rope_theta", C.c_float), ("rms_eps", C.c_float),
        ("ssm_conv_kernel", C.c_uint32), ("ssm_num_k_heads", C.c_uint32),
        ("ssm_num_v_heads", C.c_uint32), ("ssm_head_dim", C.c_uint32),
        ("full_attention_interval", C.c_uint32), ("vocab_size", C.c_uint32),
        ("mtp_layers", C.c_uint32), ("weight_sigma", C.c_float),
    ]


class TensorDesc(C.Structure):
    """Mirror of qb_tensor_desc (include/qw3b200.h)."""
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("rows", C.c_uint64), ("cols", C.c_uint64), ("data", C.c_void_p)]


def build(force=False):
    so = os.path.join(_HERE, "libqw3oracle.so")
    src = os.path.join(_HERE, "qw3_oracle.cpp")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libqw3oracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_model_create.restype = C.c_void_p
        _LIB.orc_model_create_tensors.restype = C.c_void_p
        _LIB.orc_seq_create.restype = C.c_void_p
        _LIB.orc_ksplit_policy.restype = C.c_uint32
        _LIB.orc_last_logits.restype = C.c_uint32
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def normal_table():
    t = np.empty(65536, np.float32)
    lib().orc_normal_table(_p(t))
    return t


def quantize_q8_0(w):
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty(rows * (cols // 32) * 34, np.uint8)
    lib().orc_quantize_q8_0(_p(w), C.c_uint32(rows), C.c_uint32(cols), _p(out))
    return out


def dequant_q8_0(blocks, rows, cols):
    out = np.empty((rows, cols), np.float32)
    lib().orc_dequant_q8_0(_p(blocks), C.c_uint32(rows), C.c_uint32(cols), _p(out))
    return out


def repack_split_plane(blocks, rows, cols):
    out = np.empty_like(blocks)
    lib().orc_repack_split_plane(_p(blocks), C.c_uint32(rows), C.c_uint32(cols), _p(out))
    return out


def synth_q8_0(seed, tensor_id, rows, cols, sigma=0.02):
    out = np.empty(rows * (cols // 32) * 34, np.uint8)
    lib().orc_synth_q8_0(C.c_uint64(seed), C.c_uint32(tensor_id), C.c_uint32(rows), C.c_uint32(cols),
                         C.c_float(sigma), _p(out))
    return out


def quantize_q8_1(x):
    x = _f32(x)
    M, K = x.shape
    out = np.empty(M * (K // 32) * 36, np.uint8)
    lib().orc_quantize_q8_1(_p(x), C.c_uint32(M), C.c_uint32(K), C.c_uint32(K), _p(out))
    return out


def quantize_q8_1_mmq(x):
    x = _f32(x)
    M, K = x.shape
    out = np.empty((K // 128) * M * 144, np.uint8)
    lib().orc_quantize_q8_1_mmq(_p(x), C.c_uint32(M), C.c_uint32(K), C.c_uint32(K), _p(out))
    return out


def quantize_act(x):
    """Returns (q int8 [M][K], d float32 [K/32][M])."""
    x = _f32(x)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    d = np.empty((K // 32, M), np.float32)
    lib().orc_quantize_act(_p(x), C.c_uint32(M), C.c_uint32(K), C.c_uint32(K), _p(q), _p(d))
    return q, d


def ksplit_policy(N, K):
    return int(lib().orc_ksplit_policy(C.c_uint32(N), C.c_uint32(K)))


def block_dots(blocks, N, K, q):
    M = q.shape[0]
    out = np.empty((M, N, K // 32), np.int32)
    lib().orc_block_dots(_p(blocks), C.c_uint32(N), C.c_uint32(K), _p(np.ascontiguousarray(q)), C.c_uint32(M), _p(out))
    return out


def gemm_engine(blocks, N, K, q, d, ksplit=0, want_partials=False):
    M = q.shape[0]
    S = ksplit or ksplit_policy(N, K)
    y = np.empty((M, N), np.float32)
    part = np.empty((S, M, N), np.float32) if want_partials else None
    lib().orc_gemm_engine(_p(blocks), C.c_uint32(N), C.c_uint32(K), _p(np.ascontiguousarray(q)),
                          _p(np.ascontiguousarray(d)), C.c_uint32(M), C.c_uint32(S), _p(y),
                          _p(part) if want_partials else None)
    return (y, part) if want_partials else y


def matmul_engine(blocks, N, K, x, ksplit=0):
    x = _f32(x)
    M = x.shape[0]
    y = np.empty((M, N), np.float32)
    lib().orc_matmul_engine(_p(blocks), C.c_uint32(N), C.c_uint32(K), _p(x), C.c_uint32(M), C.c_uint32(K),
                            C.c_uint32(ksplit), _p(y))
    return y


def matmul_mmvq(blocks, N, K, x):
    x = _f32(x)
    M = x.shape[0]
    xq = quantize_q8_1(x)
    y = np.empty((M, N), np.float32)
    lib().orc_matmul_mmvq(_p(blocks), C.c_uint32(N), C.c_uint32(K), _p(xq), C.c_uint32(M), _p(y))
    return y


def matmul_mmq(blocks, N, K, x):
    x = _f32(x)
    M = x.shape[0]
    xq = quantize_q8_1_mmq(x)
    y = np.empty((M, N), np.float32)
    lib().orc_matmul_mmq(_p(blocks), C.c_uint32(N), C.c_uint32(K), _p(xq), C.c_uint32(M), _p(y))
    return y


def get_rows(blocks, rows, cols, ids):
    ids = np.ascontiguousarray(ids, np.int32)
    out = np.empty((len(ids), cols), np.float32)
    lib().orc_get_rows(_p(blocks), C.c_uint32(rows), C.c_uint32(cols), _p(ids), C.c_uint32(len(ids)), _p(out))
    return out


def rms_norm(x, w, eps):
    x = _f32(x)
    M, n = x.shape
    out = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _p(_f32(w)), C.c_uint32(M), C.c_uint32(n), C.c_uint32(n), C.c_float(eps), _p(out))
    return out


def inv_freq(rope_dim, theta):
    out = np.empty(rope_dim // 2, np.float32)
    lib().orc_inv_freq(C.c_uint32(rope_dim), C.c_float(theta), _p(out))
    return out


def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, invf, n_heads, n_kv, hd, rope_dim, eps, row_seq, row_pos,
                        page_table, page_size, k_cache, v_cache):
    """In place on qkv (float32 [rows][stride]) and the uint16 caches."""
    rows, stride = qkv.shape
    lib().orc_qk_norm_rope_append(
        _p(qkv), C.c_uint32(rows), C.c_uint32(stride), _p(_f32(q_norm_w)), _p(_f32(k_norm_w)), _p(_f32(invf)),
        C.c_uint32(n_heads), C.c_uint32(n_kv), C.c_uint32(hd), C.c_uint32(rope_dim), C.c_float(eps),
        _p(row_seq), _p(row_pos), _p(page_table), C.c_uint32(page_table.shape[1]), C.c_uint32(page_size),
        _p(k_cache), _p(v_cache))


def attention_paged_gated(qkv, n_heads, n_kv, hd, row_seq, row_pos, page_table, page_size, k_cache, v_cache):
    rows, stride = qkv.shape
    out = np.empty((rows, n_heads * hd), np.float32)
    lib().orc_attention_paged_gated(
        _p(qkv), C.c_uint32(rows), C.c_uint32(stride), C.c_uint32(n_heads), C.c_uint32(n_kv), C.c_uint32(hd),
        _p(row_seq), _p(row_pos), _p(page_table), C.c_uint32(page_table.shape[1]), C.c_uint32(page_size),
        _p(k_cache), _p(v_cache), _p(out))
    return out


def deltanet_rows(proj, conv_w, ssm_a, dt_bias, norm_w, nk, nv, hd, eps, state, conv, slot_in, write_all):
    """state [n_slots][nv][hd][hd], conv [n_slots][qkv_dim][3] updated in place; returns core [T][nv*hd]."""
    T, stride = proj.shape
    core = np.empty((T, nv * hd), np.float32)
    lib().orc_deltanet_rows(
        _p(proj), C.c_uint32(T), C.c_uint32(stride), _p(_f32(conv_w)), _p(_f32(ssm_a)), _p(_f32(dt_bias)),
        _p(_f32(norm_w)), C.c_uint32(nk), C.c_uint32(nv), C.c_uint32(hd), C.c_float(eps), _p(state), _p(conv),
        C.c_uint32(state.shape[0]), C.c_uint32(slot_in), C.c_int(1 if write_all else 0), _p(core))
    return core


def argmax_rows(x):
    x = _f32(x)
    M, n = x.shape
    out = np.empty(M, np.int32)
    lib().orc_argmax_rows(_p(x), C.c_uint32(M), C.c_uint32(n), C.c_uint32(n), _p(out))
    return out


def sample_rows(logits, draft, u_acc, u_res, temp, top_p=1.0, top_k=0, min_p=0.0):
    """Per row: (token, accepted, p[draft]) of the sampling-mode acceptance; draft entries < 0 mean a plain draw."""
    x = _f32(logits)
    rows, V = x.shape
    d = np.ascontiguousarray(draft, np.int32)
    ua, ur = np.ascontiguousarray(u_acc, np.float64), np.ascontiguousarray(u_res, np.float64)
    tok, acc, pd = np.empty(rows, np.int32), np.empty(rows, np.int32), np.empty(rows, np.float32)
    lib().orc_sample_rows(_p(x), C.c_uint32(rows), C.c_uint32(V), C.c_uint32(V), _p(d), _p(ua), _p(ur), C.c_float(temp),
                          C.c_float(top_p), C.c_int32(top_k), C.c_float(min_p), _p(tok), _p(acc), _p(pd))
    return tok, acc, pd


def sampling_distribution(logits, temp, top_p=1.0, top_k=0, min_p=0.0):
    """The full-vocabulary probability vector one row is sampled from."""
    x = _f32(logits).reshape(-1)
    out = np.empty(x.size, np.float32)
    lib().orc_sampling_distribution(_p(x), C.c_uint32(x.size), C.c_float(temp), C.c_float(top_p), C.c_int32(top_k), C.c_float(min_p), _p(out))
    return out


def synth_prompt(seed, vocab, n):
    out = np.empty(n, np.int32)
    lib().orc_synth_prompt(C.c_uint64(seed), C.c_uint32(vocab), C.c_uint32(n), _p(out))
    return out


def rand_u32(seed, stream, n, i0=0):
    out = np.empty(n, np.uint32)
    lib().orc_rand_u32(C.c_uint64(seed), C.c_uint32(stream), C.c_uint64(i0), C.c_uint64(n), _p(out))
    return out


def num_threads():
    return int(lib().orc_num_threads())


class Model:
    def __init__(self, cfg, seed, max_layers=-1):
        self.cfg = cfg
        self.h = C.c_void_p(lib().orc_model_create(C.byref(cfg), C.c_uint64(seed), C.c_int32(max_layers)))

    @classmethod
    def from_tensors(cls, cfg, tensors):
        """Model from named host tensors ({GGUF name: array}: uint8 [rows][cols/32*34] = Q8_0, float32 = F32)."""
        self = cls.__new__(cls)
        self.cfg = cfg
        keep, descs = [], (TensorDesc * len(tensors))()
        for i, (name, a) in enumerate(tensors.items()):
            a = np.ascontiguousarray(a)
            nb = name.encode()
            keep += [a, nb]
            if a.dtype == np.uint8:
                descs[i] = TensorDesc(nb, 8, a.shape[0], a.shape[1] // 34 * 32, a.ctypes.data)
            else:
                assert a.dtype == np.float32, name
                descs[i] = TensorDesc(nb, 0, a.size // a.shape[-1], a.shape[-1], a.ctypes.data)
        self.h = C.c_void_p(lib().orc_model_create_tensors(C.byref(cfg), descs, C.c_size_t(len(tensors))))
        if not self.h:
            raise RuntimeError("oracle: a tensor of the model is missing or mis-shaped (see stderr)")
        return self

    def nudge_attn_norm(self, layer=0, ulps=1):
        """Moves every attn_norm gain of `layer` by `ulps` units in the last place (noise-floor measurements)."""
        lib().orc_model_nudge_attn_norm(self.h, C.c_uint32(layer), C.c_int32(ulps))

    def close(self):
        if self.h:
            lib().orc_model_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()


class Seq:
    def __init__(self, model, max_ctx):
        self.model = model
        self.h = C.c_void_p(lib().orc_seq_create(model.h, C.c_uint32(max_ctx)))

    def close(self):
        if self.h:
            lib().orc_seq_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    @property
    def position(self):
        return int(lib().orc_seq_position(self.h))

    @property
    def cur_token(self):
        return int(lib().orc_seq_cur_token(self.h))

    def set_cur_token(self, tok):
        lib().orc_seq_set_cur_token(self.h, C.c_int(int(tok)))

    def prefill(self, tokens, chunk=0):
        t = np.ascontiguousarray(tokens, np.int32)
        lib().orc_prefill(self.h, _p(t), C.c_uint32(len(t)), C.c_uint32(chunk))

    def greedy_step(self):
        return int(lib().orc_greedy_step(self.h))

    def mtp_step(self, k, forced_drafts=None):
        out = np.zeros(k + 1, np.int32)
        drafts = np.zeros(k, np.int32)
        rows = np.zeros(k + 1, np.int32)
        fd = None if forced_drafts is None else np.ascontiguousarray(forced_drafts, np.int32)
        n = lib().orc_mtp_step(self.h, C.c_uint32(k), _p(fd) if fd is not None else None, _p(out), _p(drafts), _p(rows))
        return out[:n].tolist(), drafts.tolist(), rows.tolist()

    def last_logits(self, max_rows):
        V = self.model.cfg.vocab_size
        buf = np.empty((max_rows, V), np.float32)
        r = lib().orc_last_logits(self.h, _p(buf), C.c_uint32(max_rows))
        return buf[:r]

    def forward_rows(self, tokens, want_logits=True):
        t = np.ascontiguousarray(tokens, np.int32)
        V, H = self.model.cfg.vocab_size, self.model.cfg.n_embd
        logits = np.empty((len(t), V), np.float32) if want_logits else None
        hidden = np.empty((len(t), H), np.float32)
        lib().orc_forward_rows(self.h, _p(t), C.c_uint32(len(t)), _p(logits) if want_logits else None, _p(hidden))
        return logits, hidden
