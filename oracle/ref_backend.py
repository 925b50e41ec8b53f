"""TEST INFRASTRUCTURE ONLY: ctypes wrapper over oracle/_ref/libqw3ref_backend.so, the reference's own CUDA
DeviceBackend (include/qw3/device_backend.hpp; src/kernels_cuda.cu:9564) behind the C shim ref_backend_shim.cpp.
Used by the GPU parity tests as a second comparator; never imported by the product package."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "_ref", "libqw3ref_backend.so")
# the product's DeviceBackend subclass (kvmem-qw3_b200/shim/b200_device_backend.cpp) behind the same C driver
B200_PATH = os.path.join(HERE, "_ref", "libqw3b200_backend.so")

vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int

SIG = {
    "rb_last_error": (C.c_char_p, []),
    "rb_create": (vp, [i32]),
    "rb_destroy": (None, [vp]),
    "rb_name": (C.c_char_p, [vp]),
    "rb_sync": (i32, [vp]),
    "rb_begin_capture": (i32, [vp]),
    "rb_end_capture": (i32, [vp]),
    "rb_replay_graph": (i32, [vp]),
    "rb_tensor": (vp, [vp, i32, u64]),
    "rb_tensor_free": (None, [vp]),
    "rb_tensor_elem_size": (u32, [vp]),
    "rb_upload": (i32, [vp, vp, u64, vp, u64]),
    "rb_download": (i32, [vp, vp, u64, vp, u64]),
    "rb_weight_f32": (vp, [vp, vp, u64]),
    "rb_weight_q8_0": (vp, [vp, vp, u64, u64]),
    "rb_weight_free": (None, [vp]),
    "rb_rms_norm_batch": (i32, [vp, vp, vp, vp, u32, u32, f32]),
    "rb_rmsnorm_per_head_batch": (i32, [vp, vp, vp, u32, u32, u32, u32, u32, f32]),
    "rb_rope_partial_batch": (i32, [vp, vp, u32, u32, u32, u32, u32, u32, f32]),
    "rb_kv_append_batch": (i32, [vp, vp, vp, u32, u32, u32]),
    "rb_attention_decode_batch_gated": (i32, [vp, vp, vp, u32, vp, vp, u32, u32, u32, u32, u32, u32, u32, f32]),
    "rb_recurrent_batch": (i32, [vp] * 13 + [u32] * 12 + [f32, vp, vp, u32]),
    "rb_argmax_batch": (i32, [vp, vp, u32, u32, vp, vp]),
    "rb_q8_0_matmul": (i32, [vp, vp, vp, vp, u32, u32, u32]),
    "rb_q8_0_matmul_silu_mul": (i32, [vp, vp, vp, vp, vp, u32, u32, u32]),
    "rb_q8_0_matvec_silu_mul": (i32, [vp, vp, vp, vp, vp]),
    "rb_q8_0_get_rows_batch": (i32, [vp, vp, vp, vp, u32]),
    "rb_silu_mul_n": (i32, [vp, vp, vp, vp, u64]),
    "rb_add_n": (i32, [vp, vp, vp, vp, u64]),
    "rb_kv_append_batch_paged_device": (i32, [vp, vp, vp, u32, u32, u32, vp, u32, u32]),
    "rb_attention_decode_batch_paged_gated_device": (i32, [vp, vp, vp, u32, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, u32, f32]),
    "rb_q8_0_matvec": (i32, [vp, vp, vp, vp]),
    "rb_q8_0_matvec_add": (i32, [vp, vp, vp, vp]),
    "rb_argmax_to_buffer_roundtrip": (i32, [vp, vp, u32, u32, vp, vp]),
    "rb_pack_mtp_concat": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32]),
    "rb_pack_mtp_prefix_hinputs": (i32, [vp, vp, vp, vp, u32, u32]),
    "rb_rms_norm_q8_0_matmul_fanout2": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, vp, vp, u32, u32, f32]),
}


def available():
    return os.path.exists(PATH)


class RefError(RuntimeError):
    pass


class RefBackend:
    """One reference backend instance (its own stream, cuBLAS handle and allocations)."""

    def __init__(self, linear=1, path=PATH):
        self.L = C.CDLL(path)
        for name, (res, args) in SIG.items():
            fn = getattr(self.L, name, None)
            if fn is None:                       # a library built from an older driver source
                continue
            fn.restype, fn.argtypes = res, args
        self.h = self.L.rb_create(linear)
        if not self.h:
            raise RefError(self.L.rb_last_error().decode())
        self._tensors, self._weights = [], []

    def _check(self, rc):
        if rc:
            raise RefError(self.L.rb_last_error().decode())

    def name(self):
        return self.L.rb_name(self.h).decode()

    # kind: 0 = f32, 1 = f16, 2 = i32
    def empty(self, count, kind=0):
        t = self.L.rb_tensor(self.h, kind, int(count))
        if not t:
            raise RefError(self.L.rb_last_error().decode())
        self._tensors.append(t)
        return t

    def tensor(self, arr, kind=0):
        arr = np.ascontiguousarray(arr)
        t = self.empty(arr.size, kind)
        assert self.L.rb_tensor_elem_size(t) == arr.dtype.itemsize, "tensor storage differs from the host dtype"
        self._check(self.L.rb_upload(self.h, t, 0, arr.ctypes.data, arr.nbytes))
        return t

    def download(self, t, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        self._check(self.L.rb_download(self.h, t, 0, out.ctypes.data, out.nbytes))
        return out

    def weight_f32(self, arr):
        arr = np.ascontiguousarray(arr, np.float32)
        w = self.L.rb_weight_f32(self.h, arr.ctypes.data, arr.size)
        if not w:
            raise RefError(self.L.rb_last_error().decode())
        self._weights.append(w)
        return w

    def weight_q8_0(self, blocks, rows, cols):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        w = self.L.rb_weight_q8_0(self.h, blocks.ctypes.data, rows, cols)
        if not w:
            raise RefError(self.L.rb_last_error().decode())
        self._weights.append(w)
        return w

    def call(self, name, *args):
        self._check(getattr(self.L, "rb_" + name)(self.h, *args))

    def sync(self):
        self._check(self.L.rb_sync(self.h))

    def time_us(self, op, reps=20, replays=10):
        """Device time of one `op()` in microseconds: `reps` calls captured into the backend's CUDA graph, the graph
        replayed `replays` times, wall clock around replay + synchronize (inputs stay where they are: warm L2)."""
        import time
        op()                                   # workspaces are allocated outside the capture
        self.sync()
        self._check(self.L.rb_begin_capture(self.h))
        for _ in range(reps):
            op()
        self._check(self.L.rb_end_capture(self.h))
        self._check(self.L.rb_replay_graph(self.h))
        self.sync()
        best = float("inf")
        for _ in range(replays):
            t0 = time.perf_counter()
            self._check(self.L.rb_replay_graph(self.h))
            self.sync()
            best = min(best, time.perf_counter() - t0)
        return best / reps * 1e6

    def release(self):
        self.sync()
        for t in self._tensors:
            self.L.rb_tensor_free(t)
        for w in self._weights:
            self.L.rb_weight_free(w)
        self._tensors, self._weights = [], []

    def close(self):
        if self.h:
            self.release()
            self.L.rb_destroy(self.h)
            self.h = None
