"""TEST INFRASTRUCTURE ONLY.  Two things the sampling pin needs:

* MT64: a replay of std::mt19937_64 and of libstdc++'s std::uniform_real_distribution<double>(0, 1) /
  std::discrete_distribution draw on it (generate_canonical<double, 53>: one 64-bit engine output, converted to double,
  divided by 2^64, clamped below 1), so that a test can hand the product the very draws the reference's loops would
  make (src/qwen_native_backend.cpp:423, :448 accept test; :378-379 residual / bonus / first-token draw);
* RefSampler: ctypes wrapper over oracle/_ref/libqw3ref_sampling.so, the reference's own sampler functions compiled
  from src/qwen_native_backend.cpp where it lies (ref_sampling_shim.cpp).  Never imported by the product package."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "_ref", "libqw3ref_sampling.so")
_M64 = (1 << 64) - 1


class MT64:
    """std::mt19937_64 (the 64-bit Mersenne twister of Matsumoto and Nishimura: n 312, m 156, r 31)."""
    N, M = 312, 156
    A, UM, LM = 0xB5026F5AA96619E9, 0xFFFFFFFF80000000, 0x7FFFFFFF

    def __init__(self, seed=5489):
        mt = [0] * self.N
        mt[0] = seed & _M64
        for i in range(1, self.N):
            mt[i] = (6364136223846793005 * (mt[i - 1] ^ (mt[i - 1] >> 62)) + i) & _M64
        self.mt, self.i, self.count = mt, self.N, 0

    def _twist(self):
        mt, N, M = self.mt, self.N, self.M
        for k in range(N):
            y = (mt[k] & self.UM) | (mt[(k + 1) % N] & self.LM)
            mt[k] = mt[(k + M) % N] ^ (y >> 1) ^ (self.A if y & 1 else 0)
        self.i = 0

    def next_u64(self):
        if self.i >= self.N:
            self._twist()
        y = self.mt[self.i]
        self.i += 1
        self.count += 1
        y ^= (y >> 29) & 0x5555555555555555
        y ^= (y << 17) & 0x71D67FFFEDA60000
        y ^= (y << 37) & 0xFFF7EEE000000000
        y ^= y >> 43
        return y & _M64

    def discard(self, n):
        for _ in range(n):
            self.next_u64()

    def unit(self):
        """One draw of uniform_real_distribution<double>(0, 1) / of discrete_distribution's internal uniform."""
        u = float(self.next_u64()) / 18446744073709551616.0
        return u if u < 1.0 else float(np.nextafter(1.0, 0.0))

    def random(self, size=None):
        """numpy.random.Generator-shaped access, so a DrawQueue can sit on this generator."""
        if size is None:
            return self.unit()
        n = int(np.prod(size))
        return np.array([self.unit() for _ in range(n)], np.float64).reshape(size)


def available():
    return os.path.exists(PATH)


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(PATH)
        vp, u32, u64, f32, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int32
        L.rs_distribution.argtypes = [vp, u32, f32, f32, i32, f32, f32, f32, vp, u32, vp]
        L.rs_sample_tokens.argtypes = [vp, u32, u32, f32, f32, i32, f32, u64, u64, vp, vp]
        L.rs_spec_accept.argtypes = [vp, u32, u32, vp, f32, f32, i32, f32, f32, f32, vp, u32, u64, u64, vp, vp]
        L.rs_unit_draws.argtypes = [u64, u64, u32, vp]
        for f in (L.rs_distribution, L.rs_sample_tokens, L.rs_spec_accept, L.rs_unit_draws):
            f.restype = None
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def distribution(logits, temp, top_p=1.0, top_k=0, min_p=0.0, presence=0.0, repetition=1.0, seen=()):
    x = np.ascontiguousarray(logits, np.float32).reshape(-1)
    s = np.ascontiguousarray(sorted(seen), np.uint32)
    out = np.empty(x.size, np.float32)
    lib().rs_distribution(_p(x), x.size, temp, top_p, top_k, min_p, presence, repetition, _p(s), s.size, _p(out))
    return out


def sample_tokens(logits, temp, top_p, top_k, min_p, seed, skip=0):
    x = np.ascontiguousarray(logits, np.float32)
    count, n = x.shape
    tok = np.empty(count, np.int32)
    used = C.c_uint64(0)
    lib().rs_sample_tokens(_p(x), count, n, temp, top_p, top_k, min_p, seed, skip, _p(tok), C.byref(used))
    return tok, int(used.value)


def spec_accept(rows, drafts, temp, top_p, top_k, min_p, presence, repetition, seen, seed, skip=0):
    """(accepted, extra token, engine outputs consumed) of one speculative_accept_pointmass call."""
    x = np.ascontiguousarray(rows, np.float32)
    d = np.ascontiguousarray(drafts, np.uint32)
    assert x.shape[0] == d.size + 1
    s = np.ascontiguousarray(sorted(seen), np.uint32)
    res = np.empty(2, np.int32)
    used = C.c_uint64(0)
    lib().rs_spec_accept(_p(x), d.size, x.shape[1], _p(d), temp, top_p, top_k, min_p, presence, repetition, _p(s), s.size, seed, skip,
                         _p(res), C.byref(used))
    return int(res[0]), int(res[1]), int(used.value)


def unit_draws(seed, skip, count):
    out = np.empty(count, np.float64)
    lib().rs_unit_draws(seed, skip, count, _p(out))
    return out
