"""ctypes binding of libqw3b200.so — the C ABI declared in include/qw3b200.h.

The library is CUDA-only: loading works anywhere, but creating a context without a B200 raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqw3b200.so")
_LIB = None

u32, u64, i32, f32, vp, sz = C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_void_p, C.c_size_t


class ModelConfig(C.Structure):
    """qb_model_config (include/qw3b200.h); field meaning follows the reference's QwenConfig."""
    _fields_ = [
        ("n_layers", u32), ("n_embd", u32), ("n_ff", u32), ("n_heads", u32), ("n_kv_heads", u32),
        ("head_dim", u32), ("rope_dim", u32), ("rope_theta", f32), ("rms_eps", f32),
        ("ssm_conv_kernel", u32), ("ssm_num_k_heads", u32), ("ssm_num_v_heads", u32),
        ("ssm_head_dim", u32), ("full_attention_interval", u32), ("vocab_size", u32),
        ("mtp_layers", u32), ("weight_sigma", f32),
    ]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class Sampling(C.Structure):
    """qb_sampling (include/qw3b200.h)."""
    _fields_ = [("temp", f32), ("top_p", f32), ("top_k", C.c_int32), ("min_p", f32)]


class TensorDesc(C.Structure):
    """qb_tensor_desc (include/qw3b200.h): one named host tensor of a checkpoint, GGUF type 0 (F32) or 8 (Q8_0)."""
    _fields_ = [("name", C.c_char_p), ("type", u32), ("rows", u64), ("cols", u64), ("data", vp)]


# name -> (restype, argtypes); every symbol include/qw3b200.h declares
SIGNATURES = {
    "qb_create": (i32, [i32, C.POINTER(vp)]),
    "qb_destroy": (None, [vp]),
    "qb_last_error": (C.c_char_p, []),
    "qb_synchronize": (i32, [vp]),
    "qb_stream": (vp, [vp]),
    "qb_sm_count": (i32, [vp]),
    "qb_mem_info": (i32, [vp, C.POINTER(sz), C.POINTER(sz)]),
    "qb_malloc": (i32, [vp, sz, C.POINTER(vp)]),
    "qb_free": (i32, [vp, vp]),
    "qb_memcpy_h2d": (i32, [vp, vp, vp, sz]),
    "qb_memcpy_d2h": (i32, [vp, vp, vp, sz]),
    "qb_memcpy_d2d": (i32, [vp, vp, vp, sz]),
    "qb_memset": (i32, [vp, vp, i32, sz]),
    "qb_host_alloc": (i32, [vp, sz, C.POINTER(vp)]),
    "qb_host_free": (i32, [vp, vp]),
    "qb_event_create": (i32, [vp, C.POINTER(vp)]),
    "qb_event_record": (i32, [vp, vp]),
    "qb_event_elapsed_ms": (i32, [vp, vp, vp, C.POINTER(f32)]),
    "qb_event_destroy": (i32, [vp, vp]),
    "qb_flush_l2": (i32, [vp]),
    "qb_weight_q8_0": (i32, [vp, vp, u32, u32, C.POINTER(vp)]),
    "qb_weight_q8_0_synth": (i32, [vp, u64, u32, u32, u32, f32, C.POINTER(vp)]),
    "qb_weight_q8_0_download": (i32, [vp, vp, vp]),
    "qb_weight_free": (None, [vp, vp]),
    "qb_weight_rows": (u32, [vp]),
    "qb_weight_cols": (u32, [vp]),
    "qb_quantize_q8_1": (i32, [vp, vp, u32, u32, u32, vp]),
    "qb_quantize_q8_1_mmq": (i32, [vp, vp, u32, u32, u32, vp]),
    "qb_quantize_act": (i32, [vp, vp, u32, u32, u32, vp, vp]),
    "qb_ksplit_policy": (u32, [u32, u32]),
    "qb_q8_block_dots": (i32, [vp, vp, vp, u32, vp]),
    "qb_q8_0_matmul": (i32, [vp, vp, vp, u32, u32, vp, u32, u32, i32]),
    "qb_q8_0_matmul_noalloc": (i32, [vp, vp, vp, u32, u32, vp, u32, u32]),
    "qb_q8_gemm_partials": (i32, [vp, vp, vp, vp, u32, vp, u32, i32]),
    "qb_q8_0_get_rows": (i32, [vp, vp, vp, u32, vp, u32]),
    "qb_rms_norm": (i32, [vp, vp, vp, u32, u32, u32, f32, vp]),
    "qb_qk_norm_rope_append": (i32, [vp, vp, u32, u32, vp, vp, vp, u32, u32, u32, u32, f32, vp, u32, vp, u32, u32, vp, vp]),
    "qb_attention_paged_gated": (i32, [vp, vp, u32, u32, u32, u32, u32, vp, u32, vp, u32, u32, vp, vp, u32, vp]),
    "qb_deltanet_rows": (i32, [vp, vp, u32, u32, u32, vp, vp, vp, vp, u32, u32, u32, f32, vp, vp, u32, vp, i32, vp]),
    "qb_recurrent_batch": (i32, [vp, vp, u32, vp, vp, vp, u32, vp, u32, vp, u32, vp, u32, vp, vp, vp, vp, u32, u32, u32, u32, f32, vp, vp, u32]),
    "qb_argmax_rows": (i32, [vp, vp, u32, u32, u32, vp]),
    "qb_argmax_rows_val": (i32, [vp, vp, u32, u32, u32, vp, vp, u32]),
    "qb_add": (i32, [vp, vp, vp, vp, u64]),
    "qb_mul": (i32, [vp, vp, vp, vp, u64]),
    "qb_silu": (i32, [vp, vp, vp, u64]),
    "qb_silu_mul": (i32, [vp, vp, vp, vp, u64]),
    "qb_rmsnorm_per_head": (i32, [vp, vp, vp, u32, u32, u32, u32, u32, f32]),
    "qb_rope_partial": (i32, [vp, vp, u32, u32, u32, u32, u32, u32, vp, f32]),
    "qb_kv_append": (i32, [vp, vp, vp, u32, u32, u32, vp, u32, u32]),
    "qb_apply_attn_gate": (i32, [vp, vp, vp, u32, u32, u32, u32, u32, u32]),
    "qb_attention_paged": (i32, [vp, vp, u32, u32, u32, u32, u32, vp, u32, vp, u32, u32, vp, vp, u32, vp]),
    "qb_pack_mtp_prefix_hinputs": (i32, [vp, vp, vp, vp, u32, u32]),
    "qb_pack_mtp_concat": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32]),
    "qb_model_create_synth": (i32, [vp, C.POINTER(ModelConfig), u64, C.POINTER(vp)]),
    "qb_model_create": (i32, [vp, C.POINTER(ModelConfig), C.POINTER(TensorDesc), sz, C.POINTER(vp)]),
    "qb_model_load_gguf": (i32, [vp, C.c_char_p, C.POINTER(vp), C.POINTER(ModelConfig)]),
    "qb_gguf_read_config": (i32, [C.c_char_p, C.POINTER(ModelConfig), C.POINTER(u64), C.POINTER(u64)]),
    "qb_tokenizer_load_gguf": (i32, [C.c_char_p, C.POINTER(vp)]),
    "qb_tokenizer_create": (i32, [C.POINTER(C.c_char_p), C.POINTER(u32), u32, C.POINTER(C.c_char_p), C.POINTER(u32), u32, C.c_int32, C.c_int32, i32,
                                  C.POINTER(vp)]),
    "qb_tokenizer_destroy": (None, [vp]),
    "qb_tokenizer_info": (i32, [vp, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(i32), C.POINTER(u32)]),
    "qb_tokenizer_token_id": (i32, [vp, C.c_char_p, u32]),
    "qb_tokenizer_encode": (i32, [vp, C.c_char_p, sz, i32, vp, sz, C.POINTER(sz)]),
    "qb_tokenizer_decode": (i32, [vp, vp, sz, vp, sz, C.POINTER(sz)]),
    "qb_tokenizer_split": (i32, [C.c_char_p, sz, vp, sz, C.POINTER(sz)]),
    "qb_model_get_config": (C.POINTER(ModelConfig), [vp]),
    "qb_model_create_synth_tp": (i32, [vp, C.POINTER(ModelConfig), u64, u32, u32, C.POINTER(vp)]),
    "qb_batch_set_tp": (i32, [vp, vp, vp]),
    "qb_batch_max_rows": (u32, [vp]),
    "qb_model_destroy": (None, [vp, vp]),
    "qb_model_weight_bytes": (sz, [vp]),
    "qb_batch_create": (i32, [vp, vp, u32, u32, u32, u32, i32, C.POINTER(vp)]),
    "qb_batch_create_pooled": (i32, [vp, vp, u32, u32, u32, u32, u32, C.POINTER(vp)]),
    "qb_batch_pool_info": (i32, [vp, vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]),
    "qb_seq_pages": (i32, [vp, vp, u32, vp, u32, C.POINTER(u32)]),
    "qb_prefix_capture": (i32, [vp, vp, u32, vp, u32, C.POINTER(vp)]),
    "qb_prefix_attach": (i32, [vp, vp, u32, vp]),
    "qb_prefix_tokens": (u32, [vp]),
    "qb_prefix_release": (None, [vp, vp]),
    "qb_page_pool_create": (vp, [u32]),
    "qb_page_pool_destroy": (None, [vp]),
    "qb_page_pool_alloc": (i32, [vp]),
    "qb_page_pool_share": (i32, [vp, i32]),
    "qb_page_pool_drop": (i32, [vp, i32]),
    "qb_page_pool_free_count": (u32, [vp]),
    "qb_batch_destroy": (None, [vp, vp]),
    "qb_prefill": (i32, [vp, vp, u32, vp, u32]),
    "qb_prefill_chunk": (i32, [vp, vp, u32, vp, u32]),
    "qb_prefill_sampled": (i32, [vp, vp, u32, vp, u32, C.POINTER(Sampling), C.c_double]),
    "qb_decode_greedy_step": (i32, [vp, vp]),
    "qb_mtp_draft": (i32, [vp, vp]),
    "qb_mtp_force_drafts": (i32, [vp, vp, vp, u32]),
    "qb_mtp_set_drafts": (i32, [vp, vp, vp]),
    "qb_mtp_verify": (i32, [vp, vp]),
    "qb_mtp_accept_commit": (i32, [vp, vp]),
    "qb_mtp_step": (i32, [vp, vp]),
    "qb_batch_set_draft_policy": (i32, [vp, vp, vp, i32]),
    "qb_read_step_output": (i32, [vp, vp, vp, vp]),
    "qb_batch_stats": (i32, [vp, vp, vp]),
    "qb_seq_position": (i32, [vp, vp, u32, C.POINTER(C.c_int32)]),
    "qb_seq_reset": (i32, [vp, vp, u32]),
    "qb_batch_set_active": (i32, [vp, vp, u32]),
    "qb_seq_swap": (i32, [vp, vp, u32, u32]),
    "qb_batch_set_penalties": (i32, [vp, vp, C.c_float, C.c_float]),
    "qb_batch_accept_hist": (i32, [vp, vp, vp, u32]),
    "qb_sample_rows": (i32, [vp, vp, u32, u32, u32, vp, vp, vp, C.c_float, C.c_float, i32, C.c_float, vp, vp, vp]),
    "qb_mtp_sample_rows": (i32, [vp, vp, C.c_float, C.c_float, i32, C.c_float, vp]),
    "qb_mtp_step_sampled": (i32, [vp, vp, C.c_float, C.c_float, i32, C.c_float, vp]),
    "qb_batch_snapshot": (i32, [vp, vp, C.POINTER(vp)]),
    "qb_batch_restore": (i32, [vp, vp, vp]),
    "qb_snapshot_free": (None, [vp, vp]),
    "qb_debug_last_logits": (i32, [vp, vp, vp, u32, C.POINTER(u32)]),
    "qb_debug_last_drafts": (i32, [vp, vp, vp]),
    "qb_prof_enable": (i32, [vp, i32]),
    "qb_prof_summary": (i32, [vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "qb_trace_enable": (i32, [vp, i32]),
    "qb_trace_summary": (i32, [vp, C.c_char_p, sz]),
    "qb_launch_count": (C.c_int64, [vp]),
    "qb_weight_q8_0_gate_up": (i32, [vp, vp, vp, u32, u32, C.POINTER(vp)]),
    "qb_q8_0_matmul_silu_mul_q8": (i32, [vp, vp, vp, u32, u32, vp, vp, i32]),
    "qb_tp_recv_bytes": (sz, [u32, u32, u32, u32]),
    "qb_tp_group_create": (i32, [vp, u32, u32, C.POINTER(vp), u32, u32, u32, u32, C.POINTER(vp)]),
    "qb_tp_group_destroy": (i32, [vp, vp]),
    "qb_tp_ffn_push": (i32, [vp, vp, vp, vp, vp, u32]),
    "qb_tp_ffn_reduce": (i32, [vp, vp, u32, vp, u32]),
    "qb_tp_ffn": (i32, [vp, vp, vp, vp, vp, u32, vp, u32]),
    "qb_ipc_export": (i32, [vp, vp, vp]),
    "qb_ipc_open": (i32, [vp, vp, C.POINTER(vp)]),
    "qb_ipc_close": (i32, [vp, vp]),
    "qb_debug_timeline_enable": (i32, [vp, u32]),
    "qb_debug_timeline_read": (i32, [vp, vp, vp, vp, u32, C.POINTER(u32)]),
}


class QbError(RuntimeError):
    pass


def lib():
    """Loads the CUDA library; raises if it has not been built (there is no CPU fallback)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise QbError("libqw3b200.so is missing: build it with kvmem-qw3_b200/build.py (no CPU fallback exists)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(status):
    if status != 0:
        raise QbError("qw3b200 error %d: %s" % (status, lib().qb_last_error().decode()))


def _np_ptr(a):
    return a.ctypes.data_as(vp)


class DeviceArray:
    """Device buffer with numpy-shaped host transfer."""

    def __init__(self, ctx, shape, dtype):
        self.ctx, self.shape, self.dtype = ctx, tuple(np.atleast_1d(shape)), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        p = vp()
        check(lib().qb_malloc(ctx.h, max(self.nbytes, 16), C.byref(p)))
        self.ptr = p
        ctx._arrays.append(self)   # the context keeps the buffer alive: kernels that were handed
                                   # `.ptr` may still be queued when the Python object is dropped

    @classmethod
    def from_host(cls, ctx, arr):
        arr = np.ascontiguousarray(arr)
        d = cls(ctx, arr.shape, arr.dtype)
        d.upload(arr)
        return d

    def upload(self, arr):
        arr = np.ascontiguousarray(arr, dtype=self.dtype)
        assert arr.nbytes == self.nbytes
        check(lib().qb_memcpy_h2d(self.ctx.h, self.ptr, _np_ptr(arr), self.nbytes))

    def download(self):
        out = np.empty(self.shape, self.dtype)
        check(lib().qb_memcpy_d2h(self.ctx.h, _np_ptr(out), self.ptr, self.nbytes))
        return out

    def zero(self):
        check(lib().qb_memset(self.ctx.h, self.ptr, 0, self.nbytes))

    def free(self):
        if self.ptr:
            lib().qb_free(self.ctx.h, self.ptr)
            self.ptr = None
            try:
                self.ctx._arrays.remove(self)
            except ValueError:
                pass


class Context:
    def __init__(self, device=0):
        h = vp()
        check(lib().qb_create(device, C.byref(h)))
        self.h = h
        self.device = device
        self._arrays = []

    def release_arrays(self):
        """Frees every DeviceArray created through this context."""
        for a in list(self._arrays):
            a.free()

    def close(self):
        if self.h:
            self.release_arrays()
            lib().qb_destroy(self.h)
            self.h = None

    def sync(self):
        check(lib().qb_synchronize(self.h))

    def mem_info(self):
        """(free, total) bytes of the context's device."""
        f, t = sz(), sz()
        check(lib().qb_mem_info(self.h, C.byref(f), C.byref(t)))
        return f.value, t.value

    def flush_l2(self):
        check(lib().qb_flush_l2(self.h))

    @property
    def sm_count(self):
        return lib().qb_sm_count(self.h)

    @property
    def launches(self):
        return int(lib().qb_launch_count(self.h))

    def event(self):
        e = vp()
        check(lib().qb_event_create(self.h, C.byref(e)))
        return e

    def record(self, e):
        check(lib().qb_event_record(self.h, e))

    def elapsed_ms(self, a, b):
        ms = f32()
        check(lib().qb_event_elapsed_ms(self.h, a, b, C.byref(ms)))
        return ms.value

    def prof_enable(self, on=True):
        check(lib().qb_prof_enable(self.h, 1 if on else 0))

    def prof_summary(self):
        ms, by, n = C.c_double(), C.c_double(), C.c_int64()
        check(lib().qb_prof_summary(self.h, C.byref(ms), C.byref(by), C.byref(n)))
        return dict(ms=ms.value, bytes=by.value, launches=n.value)

    def trace_enable(self, on=True):
        check(lib().qb_trace_enable(self.h, 1 if on else 0))

    def trace_summary(self):
        """[(kernel name, launches, total microseconds)] since trace_enable(True)."""
        buf = C.create_string_buffer(1 << 16)
        check(lib().qb_trace_summary(self.h, buf, len(buf)))
        out = []
        for ln in buf.value.decode().splitlines():
            n, c, t = ln.split("\t")
            out.append((n, int(c), float(t)))
        return out

    def timeline_enable(self, max_launches):
        check(lib().qb_debug_timeline_enable(self.h, max_launches))

    def timeline_read(self, max_launches):
        """Returns (stamps uint64 [n][320][4] = entry, wait passed, exit (ns), SM id; grids [n]; bytes [n])."""
        out = np.zeros((max_launches, 320, 4), np.uint64)
        grids = np.zeros(max_launches, np.uint32)
        nbytes = np.zeros(max_launches, np.float64)
        n = u32()
        check(lib().qb_debug_timeline_read(self.h, _np_ptr(out), _np_ptr(grids), _np_ptr(nbytes), max_launches, C.byref(n)))
        return out[:n.value], grids[:n.value], nbytes[:n.value]

    def timeline_gemm_summary(self, stamps, grids, nbytes):
        """In-stream figures of the recorded tensor-core GEMM launches: a launch occupies the stream from the
        moment its dependency is satisfied (earliest CTA past its wait) to its last CTA's exit; the gap before
        it is what ran between the previous GEMM's exit and that moment."""
        busy, gaps, prev_exit = 0.0, 0.0, None
        for i in range(len(grids)):
            t = stamps[i, :int(grids[i])].astype(np.int64)
            w0, x1 = int(t[:, 1].min()), int(t[:, 2].max())
            busy += (x1 - w0) * 1e-3
            if prev_exit is not None:
                gaps += max(w0 - prev_exit, 0) * 1e-3
            prev_exit = x1
        return dict(launches=int(len(grids)), busy_us=busy, gap_us=gaps, bytes=float(nbytes.sum()))

    def pinned(self, shape, dtype):
        """Pinned host array (numpy view over cudaHostAlloc memory)."""
        dt = np.dtype(dtype)
        n = int(np.prod(shape)) * dt.itemsize
        p = vp()
        check(lib().qb_host_alloc(self.h, max(n, 16), C.byref(p)))
        buf = (C.c_char * n).from_address(p.value)
        arr = np.frombuffer(buf, dtype=dt).reshape(shape)
        return arr

    def array(self, arr):
        return DeviceArray.from_host(self, arr)

    def empty(self, shape, dtype):
        return DeviceArray(self, shape, dtype)


class Weight:
    """Q8_0 weight in device layout (DeviceWeight of the reference)."""

    def __init__(self, ctx, h):
        self.ctx, self.h = ctx, h

    @classmethod
    def from_blocks(cls, ctx, blocks, rows, cols):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        assert blocks.size == rows * (cols // 32) * 34
        h = vp()
        check(lib().qb_weight_q8_0(ctx.h, _np_ptr(blocks), rows, cols, C.byref(h)))
        return cls(ctx, h)

    @classmethod
    def synth(cls, ctx, seed, tensor_id, rows, cols, sigma=0.02):
        h = vp()
        check(lib().qb_weight_q8_0_synth(ctx.h, seed, tensor_id, rows, cols, sigma, C.byref(h)))
        return cls(ctx, h)

    @property
    def rows(self):
        return lib().qb_weight_rows(self.h)

    @property
    def cols(self):
        return lib().qb_weight_cols(self.h)

    def download(self):
        out = np.empty(self.rows * (self.cols // 32) * 34, np.uint8)
        check(lib().qb_weight_q8_0_download(self.ctx.h, self.h, _np_ptr(out)))
        return out

    def free(self):
        if self.h:
            lib().qb_weight_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def act_ld(M):
    return (M + 3) & ~3


def quantize_act(ctx, x):
    """x float32 [M][K] on host -> (q DeviceArray int8 [M][K], d DeviceArray float32 [K/32][ld])."""
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    xd = ctx.array(x)
    q = ctx.empty((M, K), np.int8)
    d = ctx.empty((K // 32, act_ld(M)), np.float32)
    d.zero()
    check(lib().qb_quantize_act(ctx.h, xd.ptr, M, K, K, q.ptr, d.ptr))
    return q, d


def matmul(ctx, w, x, ksplit=0, impl=0):
    """DeviceBackend::q8_0_matmul: y[M][N] = W x, float32 host in / out."""
    x = np.ascontiguousarray(x, np.float32)
    M, K = x.shape
    N = w.rows
    xd = ctx.array(x)
    yd = ctx.empty((M, N), np.float32)
    check(lib().qb_q8_0_matmul(ctx.h, w.h, xd.ptr, M, K, yd.ptr, N, ksplit, impl))
    return yd.download()


def gguf_read_config(path):
    """(ModelConfig, number of F32 / Q8_0 tensors, their bytes) of a GGUF v3 qwen35 checkpoint; needs no GPU."""
    cfg, n, b = ModelConfig(), u64(), u64()
    check(lib().qb_gguf_read_config(os.fsencode(path), C.byref(cfg), C.byref(n), C.byref(b)))
    return cfg, n.value, b.value


class Tokenizer:
    """qb_tokenizer: the checkpoint's byte-level BPE tokenizer (host only).  Texts are bytes (str is encoded as UTF-8)."""

    def __init__(self, handle):
        self.h = handle
        v, b, e, a, n = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int(), u32()
        check(lib().qb_tokenizer_info(self.h, C.byref(v), C.byref(b), C.byref(e), C.byref(a), C.byref(n)))
        self.vocab_size, self.bos_id, self.eos_id, self.add_bos_default, self.n_special = v.value, b.value, e.value, bool(a.value), n.value

    @classmethod
    def from_gguf(cls, path):
        h = vp()
        check(lib().qb_tokenizer_load_gguf(os.fsencode(path), C.byref(h)))
        return cls(h)

    @classmethod
    def from_tables(cls, tokens, merges, bos_id=0, eos_id=0, add_bos=False):
        """tokens / merges: sequences of bytes (id = index, rank = index; a merge line is b"left right")."""
        def table(items):
            arr = (C.c_char_p * max(1, len(items)))(*items)
            lens = (u32 * max(1, len(items)))(*[len(x) for x in items])
            return arr, lens
        ta, tl = table(list(tokens))
        ma, ml = table(list(merges))
        h = vp()
        check(lib().qb_tokenizer_create(ta, tl, len(tokens), ma, ml, len(merges), bos_id, eos_id, int(add_bos), C.byref(h)))
        return cls(h)

    @staticmethod
    def _bytes(text):
        return text.encode("utf-8") if isinstance(text, str) else bytes(text)

    def encode(self, text, add_bos=False):
        raw = self._bytes(text)
        out = np.empty(len(raw) + 1, np.int32)
        n = sz()
        check(lib().qb_tokenizer_encode(self.h, raw, len(raw), int(add_bos), _np_ptr(out), out.size, C.byref(n)))
        return out[:n.value].copy()

    def decode(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        n = sz()
        cap = 64
        while True:
            buf = C.create_string_buffer(cap)
            st = lib().qb_tokenizer_decode(self.h, _np_ptr(ids), ids.size, buf, cap, C.byref(n))
            if st == 0:
                return buf.raw[:n.value]
            if n.value <= cap:
                check(st)
            cap = n.value

    def token_id(self, token):
        raw = self._bytes(token)
        return int(lib().qb_tokenizer_token_id(self.h, raw, len(raw)))

    @staticmethod
    def split(text):
        """Pieces of a text without special tokens (the split pattern alone), as bytes."""
        raw = Tokenizer._bytes(text)
        ends = np.empty(len(raw) + 1, np.uint32)
        n = sz()
        check(lib().qb_tokenizer_split(raw, len(raw), _np_ptr(ends), ends.size, C.byref(n)))
        out, b = [], 0
        for e in ends[:n.value].tolist():
            out.append(raw[b:e])
            b = e
        return out

    def close(self):
        if self.h:
            lib().qb_tokenizer_destroy(self.h)
            self.h = None


def tensor_descs(tensors):
    """tensors: {name: numpy array}; float32 arrays are F32 tensors (any shape, cols = last axis), uint8 arrays of
    shape [rows][cols/32*34] are Q8_0 block rows.  Returns (ctypes array, keep-alive list)."""
    keep, descs = [], (TensorDesc * len(tensors))()
    for i, (name, a) in enumerate(tensors.items()):
        a = np.ascontiguousarray(a)
        keep.append(a)
        if a.dtype == np.uint8:
            assert a.ndim == 2 and a.shape[1] % 34 == 0, name
            rows, cols, typ = a.shape[0], a.shape[1] // 34 * 32, 8
        else:
            assert a.dtype == np.float32, name
            cols = a.shape[-1]
            rows, typ = a.size // cols, 0
        nb = name.encode()
        keep.append(nb)
        descs[i] = TensorDesc(nb, typ, rows, cols, a.ctypes.data)
    return descs, keep


class Model:
    def __init__(self, ctx, cfg, seed):
        self.ctx, self.cfg = ctx, cfg
        h = vp()
        check(lib().qb_model_create_synth(ctx.h, C.byref(cfg), seed, C.byref(h)))
        self.h = h

    @classmethod
    def synth_tp(cls, ctx, cfg, seed, rank, world):
        """The seeded model with its FFN pairs sharded: this rank's part of `world`."""
        self = cls.__new__(cls)
        self.ctx, self.cfg = ctx, cfg
        h = vp()
        check(lib().qb_model_create_synth_tp(ctx.h, C.byref(cfg), seed, rank, world, C.byref(h)))
        self.h = h
        return self

    @classmethod
    def from_tensors(cls, ctx, cfg, tensors):
        """Model from the caller's host tensors ({GGUF tensor name: numpy array}, see tensor_descs)."""
        self = cls.__new__(cls)
        self.ctx, self.cfg = ctx, cfg
        descs, keep = tensor_descs(tensors)
        h = vp()
        check(lib().qb_model_create(ctx.h, C.byref(cfg), descs, len(tensors), C.byref(h)))
        del keep
        self.h = h
        return self

    @classmethod
    def from_gguf(cls, ctx, path):
        self = cls.__new__(cls)
        self.ctx = ctx
        h, cfg = vp(), ModelConfig()
        check(lib().qb_model_load_gguf(ctx.h, os.fsencode(path), C.byref(h), C.byref(cfg)))
        self.h, self.cfg = h, cfg
        return self

    @property
    def weight_bytes(self):
        return int(lib().qb_model_weight_bytes(self.h))

    def close(self):
        if self.h:
            lib().qb_model_destroy(self.ctx.h, self.h)
            self.h = None


class Batch:
    """Executor state of n_seqs requests (the QwenExecutor-side state of the reference)."""

    def __init__(self, model, n_seqs, max_ctx, k, page_size=16, page_order=0, pool_pages=0):
        """pool_pages > 0: the pooled form (one K/V page pool shared by the sequences, pages handed out as positions grow)."""
        self.ctx, self.model, self.n_seqs, self.k, self.max_ctx = model.ctx, model, n_seqs, k, max_ctx
        self.n_active = n_seqs
        self.page_size, self.pool_pages = page_size, pool_pages
        h = vp()
        if pool_pages:
            check(lib().qb_batch_create_pooled(self.ctx.h, model.h, n_seqs, max_ctx, k, page_size, pool_pages, C.byref(h)))
        else:
            check(lib().qb_batch_create(self.ctx.h, model.h, n_seqs, max_ctx, k, page_size, page_order, C.byref(h)))
        self.h = h
        self._n = np.zeros(n_seqs, np.int32)
        self._t = np.zeros((n_seqs, k + 1), np.int32)

    def close(self):
        if self.h:
            lib().qb_batch_destroy(self.ctx.h, self.h)
            self.h = None

    def pool_info(self):
        f, t, ps = u32(), u32(), u32()
        check(lib().qb_batch_pool_info(self.ctx.h, self.h, C.byref(f), C.byref(t), C.byref(ps)))
        return dict(free=f.value, total=t.value, page_size=ps.value)

    def seq_pages(self, seq):
        n = u32()
        out = np.zeros(4096, np.int32)
        check(lib().qb_seq_pages(self.ctx.h, self.h, seq, _np_ptr(out), out.size, C.byref(n)))
        return out[:n.value].tolist()

    def prefix_capture(self, seq, tokens=None):
        """An entry of the prefix cache from sequence `seq`, which must stand at the end of a prefill(..., more=True)."""
        t = None if tokens is None else np.ascontiguousarray(tokens, np.int32)
        h = vp()
        check(lib().qb_prefix_capture(self.ctx.h, self.h, seq, _np_ptr(t) if t is not None else None, 0 if t is None else len(t), C.byref(h)))
        return h

    def prefix_attach(self, seq, prefix):
        check(lib().qb_prefix_attach(self.ctx.h, self.h, seq, prefix))

    def prefix_release(self, prefix):
        lib().qb_prefix_release(self.ctx.h, prefix)

    def prefill(self, seq, tokens, more=False):
        """Ingests prompt tokens of sequence `seq`; more=True: the prompt continues in a later call (no token is chosen)."""
        t = np.ascontiguousarray(tokens, np.int32)
        fn = lib().qb_prefill_chunk if more else lib().qb_prefill
        check(fn(self.ctx.h, self.h, seq, _np_ptr(t), len(t)))

    def prefill_sampled(self, seq, tokens, u, temp, top_p=1.0, top_k=0, min_p=0.0):
        """The end of a sampled request's prompt: the first token is drawn with the uniform draw u."""
        t = np.ascontiguousarray(tokens, np.int32)
        sp = Sampling(temp, top_p, top_k, min_p)
        check(lib().qb_prefill_sampled(self.ctx.h, self.h, seq, _np_ptr(t), len(t), C.byref(sp), float(u)))

    def greedy_step(self):
        check(lib().qb_decode_greedy_step(self.ctx.h, self.h))

    def mtp_draft(self):
        check(lib().qb_mtp_draft(self.ctx.h, self.h))

    def mtp_force_drafts(self, forced_dev, stride):
        """forced_dev: DeviceArray int32 [n_seqs][stride]; draft i becomes forced[pos + 1 + i]."""
        check(lib().qb_mtp_force_drafts(self.ctx.h, self.h, forced_dev.ptr, stride))

    def mtp_set_drafts(self, drafts_host):
        """drafts_host: int32 numpy array [n_seqs][k] (pinned for an asynchronous copy)."""
        check(lib().qb_mtp_set_drafts(self.ctx.h, self.h, _np_ptr(drafts_host)))

    def mtp_verify(self):
        check(lib().qb_mtp_verify(self.ctx.h, self.h))

    def mtp_accept_commit(self):
        check(lib().qb_mtp_accept_commit(self.ctx.h, self.h))

    def mtp_step(self):
        check(lib().qb_mtp_step(self.ctx.h, self.h))

    def set_draft_policy(self, limits=None, eos_token=-1):
        """limits: per-sequence draft depth of the next steps (None = k everywhere); eos_token ends a chain when drafted."""
        lim = None if limits is None else np.ascontiguousarray(limits, np.int32)
        check(lib().qb_batch_set_draft_policy(self.ctx.h, self.h, _np_ptr(lim) if lim is not None else None, int(eos_token)))

    def set_tp(self, group):
        """Run the FFN blocks through a tensor-parallel group (tp.TpGroup) or back on one GPU (None)."""
        check(lib().qb_batch_set_tp(self.ctx.h, self.h, group.h if group is not None else None))

    @property
    def max_rows(self):
        return int(lib().qb_batch_max_rows(self.h))

    def set_penalties(self, presence=0.0, repetition=1.0):
        check(lib().qb_batch_set_penalties(self.ctx.h, self.h, presence, repetition))

    def mtp_step_sampled(self, u, temp, top_p=1.0, top_k=0, min_p=0.0):
        """u: float64 [n_seqs][k+1] uniform draws (see qb_mtp_sample_rows)."""
        u = np.ascontiguousarray(u, np.float64).reshape(self.n_seqs, self.k + 1)
        check(lib().qb_mtp_step_sampled(self.ctx.h, self.h, temp, top_p, top_k, min_p, _np_ptr(u)))

    def mtp_sample_rows(self, u, temp, top_p=1.0, top_k=0, min_p=0.0):
        u = np.ascontiguousarray(u, np.float64).reshape(self.n_seqs, self.k + 1)
        check(lib().qb_mtp_sample_rows(self.ctx.h, self.h, temp, top_p, top_k, min_p, _np_ptr(u)))

    def read_output(self):
        """Returns a list (per sequence) of the tokens the last step emitted."""
        check(lib().qb_read_step_output(self.ctx.h, self.h, _np_ptr(self._n), _np_ptr(self._t)))
        return [self._t[s, :self._n[s]].tolist() for s in range(self.n_seqs)]

    def stats(self):
        out = np.zeros(4, np.int64)
        check(lib().qb_batch_stats(self.ctx.h, self.h, _np_ptr(out)))
        return dict(steps=int(out[0]), drafted=int(out[1]), accepted=int(out[2]), emitted=int(out[3]))

    def accept_hist(self):
        """(steps that rejected a draft, [steps that accepted exactly a drafts for a = 0 .. k])."""
        out = np.zeros(self.k + 2, np.int64)
        check(lib().qb_batch_accept_hist(self.ctx.h, self.h, _np_ptr(out), out.size))
        return int(out[0]), [int(v) for v in out[1:]]

    def spec_summary_lines(self):
        """The speculative loop's counters in the form of the reference's log lines (native mtp_spec_summary: and
        native mtp_accept_hist:, src/qwen_native_backend.cpp:16313-16392), so that its log parsers keep working; fields
        this engine has no counterpart for (adaptive policy, per-phase host timers) carry their neutral values."""
        st = self.stats()
        rejected, hist = self.accept_hist()
        acc = st["accepted"] / st["drafted"] if st["drafted"] else 0.0
        summary = ("native mtp_spec_summary: enabled=true batches=%d drafted=%d accepted=%d rejected=%d rollbacks=%d adaptive=false "
                   "promotions=0 reject_budget=off fallback=false acceptance=%.4f state_ckpt_count=%d batched_verify_batches=%d "
                   "batched_verify_tokens=%d" % (st["steps"], st["drafted"], st["accepted"], rejected, rejected, acc, self.k,
                                                  st["steps"], st["steps"] * (self.k + 1)))
        return [summary, "native mtp_accept_hist:" + "".join(" len%d=%d" % (a, n) for a, n in enumerate(hist))]

    def reset(self, seq):
        """Retire the request in slot `seq`: position 0, zero recurrent state; prefill admits the next one."""
        check(lib().qb_seq_reset(self.ctx.h, self.h, seq))

    def set_active(self, n):
        """The decode steps run the sequences [0, n)."""
        check(lib().qb_batch_set_active(self.ctx.h, self.h, n))
        self.n_active = n

    def swap(self, s1, s2):
        check(lib().qb_seq_swap(self.ctx.h, self.h, s1, s2))

    def snapshot(self):
        """Opaque snapshot of every sequence's state (see qb_batch_snapshot); free with free_snapshot."""
        h = vp()
        check(lib().qb_batch_snapshot(self.ctx.h, self.h, C.byref(h)))
        return h

    def restore(self, snap):
        check(lib().qb_batch_restore(self.ctx.h, self.h, snap))

    def free_snapshot(self, snap):
        lib().qb_snapshot_free(self.ctx.h, snap)

    def position(self, seq):
        p = C.c_int32()
        check(lib().qb_seq_position(self.ctx.h, self.h, seq, C.byref(p)))
        return p.value

    def last_drafts(self):
        out = np.zeros((self.n_seqs, self.k), np.int32)
        check(lib().qb_debug_last_drafts(self.ctx.h, self.h, _np_ptr(out)))
        return out

    def last_logits(self, max_rows):
        V = self.model.cfg.vocab_size
        buf = np.empty((max_rows, V), np.float32)
        r = u32()
        check(lib().qb_debug_last_logits(self.ctx.h, self.h, _np_ptr(buf), max_rows, C.byref(r)))
        return buf[:r.value]
